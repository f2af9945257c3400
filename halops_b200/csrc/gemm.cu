// Block-scaled dense GEMM for sm_100a: out[M,N] = bf16(alpha * A[M,K] . B[N,K]^T)
// with MXFP8 (e4m3 + UE8M0 / 32), NVFP4 (e2m1 + UE4M3 / 16) or MXFP4 (e2m1 +
// UE8M0 / 32) operands whose scales arrive in the 128x4 SfAtom order.
//
// Replaces the reference's CUTLASS/CuTe kernel (csrc/kernel/gemm/gemm_kernel.cuh:28-285,
// mainloop_fwd.cuh:405-1007, epilogue.cuh:713-1058, tile_scheduler.cuh:523-542)
// with hand-written PTX.  Per CTA (one per SM, persistent over output tiles):
//   warp 0   TMA producer: A and B tiles (128-byte swizzle) by tensor map, the
//            512-byte scale atoms by flat bulk copies, into a ring of stages
//   warp 1   one thread issues the block-scaled tcgen05.mma (fp32 accumulators
//            in tensor memory, two accumulator stages so the epilogue overlaps
//            the next tile)
//   warps 2-5 epilogue: tcgen05.ld -> * alpha -> bf16 -> swizzled staging in
//            shared memory -> TMA store (rows >= M are dropped by the tensor
//            map extent, so neither A nor the output is ever padded)
//   warps 6-9 scales: shared memory -> registers -> tensor memory (tcgen05.st),
//            one warp per lane quarter, a few k-tiles ahead of the MMAs
//   warp 10  64-wide dense tiles only: a second MMA issuer that takes every other
//            k-tile into an accumulator of its own (the epilogue adds the two); one
//            thread needs about 600 cycles to issue and commit a k-tile of 8 KB
// Every mbarrier wait is bounded: a role that waits longer than kTimeoutNs
// records a code in the device status word, raises the CTA's abort flag and
// all roles leave through the common teardown that frees tensor memory.

#include <cuda_bf16.h>

#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace hq {
namespace {

constexpr int kBM = 128;           // rows of A per CTA tile
constexpr int kBKBytes = 128;      // bytes of K per stage row: 128 e4m3 or 256 e2m1
constexpr int kThreads = 352;      // single-CTA kernel: 11 warps (pair kernel: see Cfg2)
constexpr int kEpiWarps = 4;
constexpr int kSfWarps = 4;        // single-CTA kernel: warps 6-9 move the scales into tensor memory
constexpr int kEpiChunk = 32;      // accumulator columns per tcgen05.ld / TMA store
constexpr int kEpiBufBytes = 32 * kEpiChunk * 2;  // 32 rows x 64 bytes
constexpr uint64_t kTimeoutNs = 2000000000ull;    // bound of every device-side wait
constexpr int kSmemBudget = 232448;               // 227 KiB opt-in maximum per CTA

// device status word: non-zero when a kernel gave up on a bounded wait
__device__ uint32_t g_status[4];

enum : uint32_t {
    kStatusProducer = 0x01,
    kStatusMma = 0x02,
    kStatusEpilogue = 0x04,
};

template <int BN, int KIND>
struct Cfg {
    static_assert(BN == 64 || BN == 128 || BN == 256, "tile widths built");
    static constexpr int kABytes = kBM * kBKBytes;
    static constexpr int kBBytes = BN * kBKBytes;
    // SfAtoms along K that one stage needs per 128 rows: K elements per stage / (4 * group)
    static constexpr int kSfKAtoms = (KIND == 0 || KIND == 3) ? 1 : (KIND == 1 ? 4 : 2);
    static constexpr int kNAtoms = (BN + 127) / 128;
    static constexpr int kSfaBytes = kSfKAtoms * 512;
    static constexpr int kSfbBytes = kNAtoms * kSfaBytes;
    static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
    static constexpr int kEpiBufs = (KIND == 1 && BN == 256) ? 1 : 2;
    static constexpr int kEpiBytes = kEpiWarps * kEpiBufs * kEpiBufBytes;
    static constexpr int kBarBytes = 1024;
    static constexpr int kStagesFit = (kSmemBudget - kEpiBytes - kBarBytes - 1024) / kStageBytes;
    static constexpr int kStages = kStagesFit > 8 ? 8 : kStagesFit;
    static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + kBarBytes + 1024;

    // Tensor memory columns: two accumulator stages of BN columns, then kSfSets sets of scale
    // columns (one set = the scales of one k-tile: kSfKAtoms * 4 columns for A, then
    // kSfKAtoms * kNAtoms * 4 for B).  When BN == 256 the accumulator stages overlap by
    // kOverlap columns so that everything fits in 512 (the epilogue drains the shared
    // columns first).  The scales are written by four warps of their own (tcgen05.st, one
    // warp per lane quarter) into the set it % kSfSets, so they run ahead of the MMAs: a
    // tcgen05.cp of one 512-byte atom occupies the copy unit for 75-90 cycles whoever issues
    // it, and NVFP4 needs 12 per k-tile of 512 MMA cycles.
    static constexpr int kSfCols = kSfKAtoms * 4 * (1 + kNAtoms);
    static constexpr int kSfSets = BN < 256 ? 4 : 2;
    static constexpr int kSfRegion = kSfCols * kSfSets;
    static constexpr int kOverlap = BN == 256 ? (kSfRegion + 15) / 16 * 16 : 0;
    static constexpr int kAccStride = BN - kOverlap;
    static constexpr int kSfaCol = kAccStride + BN;  // set 0
    static constexpr int kSfbCol = kSfaCol + kSfKAtoms * 4;
    // 64-wide tiles: two more accumulator stages, for the second MMA issuer (behind the scales)
    static constexpr int kDualCol = kSfaCol + kSfRegion;
    static constexpr int kColsUsed = kDualCol + (BN == 64 ? 2 * BN : 0);
    static constexpr int kTmemCols = kColsUsed <= 32 ? 32 : kColsUsed <= 64 ? 64 : kColsUsed <= 128 ? 128
                                     : kColsUsed <= 256 ? 256 : 512;
    static_assert(kColsUsed <= 512, "tensor memory budget");
    static constexpr int kChunks = BN / kEpiChunk;
    static constexpr int kOverlapChunks = (kOverlap + kEpiChunk - 1) / kEpiChunk;
    static_assert(kStages >= 2, "pipeline depth");
};

struct Barriers {
    uint64_t full[16];
    uint64_t empty[16];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t overlap_free[2];
    uint64_t sf_full[16];  // single-CTA kernel: the scale bytes of a stage have landed
    uint64_t sf_ready[4];  // the scales of a k-tile are in tensor memory
    uint64_t turn[2];      // pair kernel: hands the MMA issue from one issuer thread to the other
    uint64_t recv_full;    // split-K: the other CTA's partial sums have landed in this CTA's buffer
    uint64_t epi_sync;     // small-M kernel: rendezvous of the four epilogue warps (a bounded wait, unlike bar.sync)
    uint32_t tmem_base;
    uint32_t abort;
};

// Bounded mbarrier wait.  Returns false when the CTA is aborting.
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile uint32_t* abort,
                                         uint32_t code, uint64_t limit_ns = kTimeoutNs) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = ptx::globaltimer_ns();
    uint32_t spins = 0;
    while (!ptx::mbar_try_wait(bar, parity)) {
        if ((++spins & 31u) == 0u) {
            if (*abort != 0u) return false;
            if (ptx::globaltimer_ns() - t0 > limit_ns) {
                *abort = 1u;
                atomicOr(&g_status[0], code);
                return false;
            }
        }
    }
    return true;
}

struct TileCoord {
    int m;
    int n;
};

// Persistent static schedule: tile ids walk down groups of 8 row tiles, then
// across columns, so one wave of CTAs shares a small set of A and B tiles in L2.
__device__ __forceinline__ TileCoord tile_coord(int tile, int tiles_m, int tiles_n) {
    constexpr int kGroup = 8;
    if (tiles_m == 1) return {0, tile};  // decode shapes: no divisions on the way to the first load
    const int per_group = kGroup * tiles_n;
    const int g = tile / per_group;
    const int first_m = g * kGroup;
    const int gsz = min(kGroup, tiles_m - first_m);
    const int r = tile - g * per_group;
    return {first_m + r % gsz, r / gsz};
}

// How the rows of A map to weights.  Dense: one weight.  The grouped kinds stack
// `count` weights [count, N, K] (scales: every weight starts on its own 128-row atom):
//   batch       A rows [g * rows, (g + 1) * rows) use weight g; out is [rows, count * N]
//   masked      the same slots, of which only the first table[g] rows are valid;
//               out is [count * rows, N]
//   contiguous  row r uses weight table[r] (sorted, every run of equal ids starts on a
//               multiple of 64 rows); out is [M, N]
// Follows the reference's four kernel modes (csrc/kernel/gemm/tile_scheduler.cuh:253-297,
// 393-460, 575-670).
enum { kGroupDense = 0, kGroupBatch = 1, kGroupMasked = 2, kGroupContiguous = 3 };

struct GroupParams {
    int kind;
    int count;         // number of weights
    int rows;          // rows per batch / padded rows per expert (batch, masked)
    const int* table;  // masked: valid rows per expert; contiguous: expert of every row
};

// What one persistent-loop iteration of the single-CTA kernel works on.
struct Work {
    int a_row0;     // first row of the A box (and 128 x its scale-atom row)
    int b_row0;     // first row of the B box in the stacked weights
    int sfb_tile;   // 128-row scale atom row of the B box
    int sfb_shift;  // 32-row group of the B box inside that atom (BN = 64 only)
    int group;      // weight index: selects alpha and the bias row
    int row_lo;     // accumulator rows [row_lo, row_hi) belong to this item; the others
    int row_hi;     //   are padding or belong to the neighbouring group
    int out_row0;   // output row of accumulator row 0 (negative when a batch starts mid-tile)
    int out_col0;   // first output column
    int bias_col0;  // first bias element
};

// The three warp roles walk the same sequence of work items, each with its own copy
// of this iterator.  Tiles are cut on 128-row boundaries of the stacked A rows (where
// the scale atoms are); a tile that holds rows of two groups is worked once per group
// (the reference's rule for batches, csrc/kernel/gemm/gemm_dispatch.cuh:90-93).
template <int BN>
struct WorkIter {
    GroupParams g;
    int M, N, tiles_m, tiles_n;
    int tile;
    int pass = 0;        // contiguous: second expert of a tile
    int walk_group = 0;  // batch / masked: group of the last item and the number of
    int walk_base = 0;   //   (group, row tile) pairs before it

    int stride;          // work items between two items of this CTA (or cluster)

    __device__ WorkIter(const GroupParams& grp, int m, int n, int tm, int tn, int first = blockIdx.x,
                        int step = gridDim.x)
        : g(grp), M(m), N(n), tiles_m(tm), tiles_n(tn), tile(first), stride(step) {}

    __device__ __forceinline__ void set_b(Work& w, int group, int nt) const {
        w.group = group;
        w.b_row0 = group * N + nt * BN;
        w.sfb_tile = group * ((N + 127) / 128) + (nt * BN) / 128;
        w.sfb_shift = ((nt * BN) % 128) / 32;
        w.bias_col0 = w.b_row0;
    }

    __device__ bool next(Work& w) {
        if (g.kind == kGroupDense || g.kind == kGroupContiguous) {
            if (tile >= tiles_m * tiles_n) return false;
            const TileCoord tc = tile_coord(tile, tiles_m, tiles_n);
            w.a_row0 = tc.m * kBM;
            w.out_row0 = w.a_row0;
            w.out_col0 = tc.n * BN;
            w.row_lo = 0;
            w.row_hi = min(kBM, M - w.a_row0);
            int group = 0;
            if (g.kind == kGroupContiguous) {
                const int e0 = __ldg(g.table + w.a_row0);
                const int e1 = w.a_row0 + 64 < M ? __ldg(g.table + w.a_row0 + 64) : e0;
                group = min(max(pass != 0 ? e1 : e0, 0), g.count - 1);
                if (e1 != e0) {
                    // two experts meet in the middle of this tile: one pass each
                    if (pass == 0) {
                        w.row_hi = 64;
                    } else {
                        w.row_lo = 64;
                    }
                    pass ^= 1;
                }
            }
            set_b(w, group, tc.n);
            if (pass == 0) tile += stride;
            return true;
        }
        // batch / masked: item = (group, j-th row tile that holds valid rows of it, n tile)
        const int pair = tile / tiles_n;
        const int nt = tile - pair * tiles_n;
        int first, valid;
        for (;;) {
            if (walk_group >= g.count) return false;
            first = walk_group * g.rows;
            valid = g.kind == kGroupMasked ? min(max(__ldg(g.table + walk_group), 0), g.rows) : g.rows;
            const int cnt = valid > 0 ? (first + valid - 1) / kBM - first / kBM + 1 : 0;
            if (pair < walk_base + cnt) break;
            walk_base += cnt;
            ++walk_group;
        }
        w.a_row0 = (first / kBM + (pair - walk_base)) * kBM;
        w.row_lo = max(0, first - w.a_row0);
        w.row_hi = min(kBM, first + valid - w.a_row0);
        set_b(w, walk_group, nt);
        if (g.kind == kGroupBatch) {
            w.out_row0 = w.a_row0 - first;
            w.out_col0 = w.b_row0;
        } else {
            w.out_row0 = w.a_row0;
            w.out_col0 = nt * BN;
        }
        tile += stride;
        return true;
    }
};

template <int BN, int KIND>
__device__ __forceinline__ uint32_t instr_desc(uint32_t sf_id) {
    // block-scaled instruction descriptor: [4,6) SFB byte id, [7,10) A format,
    // [10,13) B format, bit 15/16 A/B major (0 = K), [17,23) N >> 3,
    // bit 23 scale format (1 = UE8M0, 0 = UE4M3), [24,29) M >> 4, [29,31) SFA byte id
    // KIND 0: e4m3 x e4m3 (code 0); KIND 1 / 2: e2m1 x e2m1 of the mxf4nvf4 kinds (code 1);
    // KIND 3: e4m3 x e2m1 of the mxf8f6f4 kind, whose code for e2m1 is 5
    constexpr uint32_t fmt_a = (KIND == 0 || KIND == 3) ? 0u : 1u;
    constexpr uint32_t fmt_b = KIND == 0 ? 0u : (KIND == 3 ? 5u : 1u);
    constexpr uint32_t scale_fmt = KIND == 1 ? 0u : 1u;
    return (sf_id << 4) | (fmt_a << 7) | (fmt_b << 10) | (uint32_t(BN >> 3) << 17) | (scale_fmt << 23) |
           (uint32_t(kBM >> 4) << 24) | (sf_id << 29);
}

// Parameters of the SiTU-GLU quantising epilogue (all zero for the other epilogues).
struct SituParams {
    uint8_t* q;       // e4m3 output: [M, N/2] (SituQuant) or [M, B * N] (the batch Quant epilogues)
    uint8_t* sf;      // UE8M0 scales of the output, SfAtom order, kb_out scale columns
    int64_t ldq;      // bytes between output rows
    int kb_out;       // scale columns of the output: N / 2 / 32 or B * N / 32
    float beta;       // gate soft-cap
    float inv_beta;
    float lin;        // up soft-cap, 0 = none
    float inv_lin;
    const __nv_bfloat16* gate;  // [M, B * N] multiplier of the GateMulQuant epilogues (logits for the sigmoid form)
    int64_t gate_ld;            // elements between its rows
    int valid_rows;             // rows of the quantised output; `sf` covers them rounded up to 128
};

// The quantising epilogues store a scale byte for every row that exists.  The rows that pad
// the last 128-row SfAtom get zero bytes here (what group_wise_quant writes there), so a
// caller need not clear `sf` first.  Called by the 128 epilogue threads of every CTA.
__device__ __forceinline__ void zero_sf_padding(const SituParams& sp, int tid) {
    const int pad_rows = (128 - (sp.valid_rows & 127)) & 127;
    const int total = pad_rows * sp.kb_out;
    for (int i = int(blockIdx.x) * 128 + tid; i < total; i += int(gridDim.x) * 128) {
        const int row = sp.valid_rows + i / sp.kb_out;
        const int kb = i % sp.kb_out;
        sp.sf[(int64_t(row >> 7) * (sp.kb_out >> 2) + (kb >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 +
              (kb & 3)] = 0;
    }
}

__device__ __forceinline__ float tanh_fast(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
    return t;
}

// 16 SiTU-GLU outputs from one 32-column accumulator chunk whose first 16 columns
// are gate rows and last 16 the matching up rows (the row order interleave_gate_up
// produces): bf16(beta tanh(g / beta) sigmoid(g) * lin tanh(u / lin)), or * u when
// there is no up soft-cap (reference: halops/gemm/dense_gemm.py:100-109,
// csrc/common/activation.cuh:33-62; the sigmoid here is 0.5 tanh(g / 2) + 0.5).
__device__ __forceinline__ void situ_chunk(const uint32_t (&r)[32], const __nv_bfloat16* __restrict__ bias_chunk,
                                           const SituParams& sp, uint32_t* y8) {
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
    if (bias_chunk != nullptr) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4 b = __ldg(reinterpret_cast<const uint4*>(bias_chunk) + j);
            const uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[8 * j + 2 * i] += __uint_as_float(w[i] << 16);
                v[8 * j + 2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
            }
        }
    }
    float o[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float g = v[i];
        const float u = v[16 + i];
        const float gate = sp.beta * tanh_fast(g * sp.inv_beta) * fmaf(0.5f, tanh_fast(0.5f * g), 0.5f);
        const float up = sp.lin != 0.0f ? sp.lin * tanh_fast(u * sp.inv_lin) : u;
        o[i] = gate * up;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const __nv_bfloat162 p = __float22bfloat162_rn(make_float2(o[2 * i], o[2 * i + 1]));
        y8[i] = *reinterpret_cast<const uint32_t*>(&p);
    }
}

// MXFP8 quantisation of 32 bf16 values (16 packed words) of one row: UE8M0 byte
// e = ceil(log2(amax / 448)) + 127 computed exactly on the bf16 bit fields (floor 85),
// codes = e4m3(v * 2^(127 - e)) with NaN -> -448.  This is the exact-integer recipe of
// the reference's quantising epilogue (csrc/common/mx_quant.cuh:60-71,
// csrc/kernel/gemm/epilogue.cuh:990-1010), not the fast-math one of group_wise_quant.
__device__ __forceinline__ uint32_t quant32_bf16(const uint32_t (&y)[16], uint4& lo, uint4& hi) {
    uint32_t mx = y[0] & 0x7fff7fffu;
#pragma unroll
    for (int i = 1; i < 16; ++i) {
        uint32_t a = y[i] & 0x7fff7fffu, m2;
        asm("max.bf16x2 %0, %1, %2;" : "=r"(m2) : "r"(mx), "r"(a));
        mx = m2;
    }
    uint32_t sw = __byte_perm(mx, 0, 0x1032), m2;
    asm("max.bf16x2 %0, %1, %2;" : "=r"(m2) : "r"(mx), "r"(sw));
    const uint32_t bits = m2 & 0xffffu;                      // bf16 amax: 8 exponent, 7 mantissa bits
    const uint32_t exp8 = ((bits + 31u) >> 7) & 0xffu;       // exponent, + 1 when the mantissa exceeds 1.75
    const uint32_t e = max(exp8, 85u + 8u) - 8u;
    const float mult = __uint_as_float((254u - e) << 23);
    uint32_t c[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        uint32_t g;
        asm("max.bf16x2 %0, %1, %2;" : "=r"(g) : "r"(y[i]), "r"(0xff80ff80u));  // NaN -> -inf -> -448
        const float a = __uint_as_float(g << 16) * mult;
        const float b = __uint_as_float(g & 0xffff0000u) * mult;
        uint16_t h;
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(h) : "f"(a), "f"(b));
        c[i] = h;
    }
    lo = make_uint4(c[0] | (c[1] << 16), c[2] | (c[3] << 16), c[4] | (c[5] << 16), c[6] | (c[7] << 16));
    hi = make_uint4(c[8] | (c[9] << 16), c[10] | (c[11] << 16), c[12] | (c[13] << 16), c[14] | (c[15] << 16));
    return e;
}

// Epilogue math for one 32-column chunk of one accumulator row:
// y = acc * alpha (+ bias[col]); Identity stores bf16(y), Sigmoid stores
// bf16(0.5 * tanh.approx(0.5 * y) + 0.5), the reference's formulation
// (csrc/common/activation.cuh:25-27, csrc/kernel/gemm/epilogue.cuh:867-951).
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&r)[32], uint32_t (&p)[16], float scale,
                                               const __nv_bfloat16* __restrict__ bias_chunk, int epi_op) {
    float y[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) y[i] = __uint_as_float(r[i]) * scale;
    if (bias_chunk != nullptr) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4 b = __ldg(reinterpret_cast<const uint4*>(bias_chunk) + j);
            const uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                y[8 * j + 2 * i] += __uint_as_float(w[i] << 16);
                y[8 * j + 2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
            }
        }
    }
    if (epi_op == HQ_EPILOGUE_SIGMOID) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            float t;
            asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * y[i]));
            y[i] = fmaf(0.5f, t, 0.5f);
        }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const __nv_bfloat162 v = __float22bfloat162_rn(make_float2(y[2 * i], y[2 * i + 1]));
        p[i] = *reinterpret_cast<const uint32_t*>(&v);
    }
}

// kSplitK (64-wide tiles, one row of tiles, at most half as many tiles as SMs): a cluster of
// two CTAs works one tile, each half of the k-tiles; the second CTA sends its fp32 partial
// sums through distributed shared memory into a 32 KB buffer of the first (carved out of the
// last two A stages), which adds them to its accumulator before the usual epilogue.
template <int BN, int KIND, bool kSplitK = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
            const __grid_constant__ CUtensorMap tm_d, const uint8_t* __restrict__ sfa,
            const uint8_t* __restrict__ sfb, const float* __restrict__ alpha,
            const __nv_bfloat16* __restrict__ bias, int epi_op, __nv_bfloat16* __restrict__ out, int64_t ldo,
            int M, int N, int k_tiles, int kq_dim, int tiles_m, int tiles_n, int a_rows, int direct_store,
            int dual_issue, const GroupParams grp, const SituParams situ) {
    using C = Cfg<BN, KIND>;
    // Two MMA issuers with an accumulator each (64-wide dense tiles, plain epilogues): the k-tiles
    // of a tile are summed as (even ones) + (odd ones), deterministically, but not in the k order
    // of the other tiles.
    const bool dual = BN == 64 && !kSplitK && dual_issue == 1;
    // dual_issue == 2: two issuers as well, but into ONE accumulator and in k order, as in the
    // 2-CTA kernel: the threads take alternate k-iterations and hand each other the turn (tcgen05
    // fences around an mbarrier arrival), so the MMAs reach the tensor core in the order one thread
    // would issue them and the bits do not change.  What it buys is issue time: 4 MMAs and the
    // commit that releases the stage keep one thread busy for longer than a narrow tile's MMAs run.
    const bool ordered = dual_issue == 2;
    static_assert(!kSplitK || (BN == 64 && 2 * C::kABytes == kBM * BN * 4 && C::kStages >= 6), "split-K buffer");
    // stages of the ring; with split-K the last two A stages hold the partial sums received
    constexpr uint32_t kRing = kSplitK ? C::kStages - 2 : C::kStages;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: required by the 128-byte swizzle of the operand tiles
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* const smem = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
    const uint32_t a_base = smem_base;
    const uint32_t recv_base = a_base + kRing * C::kABytes;
    const uint32_t k_rank = kSplitK ? ptx::cluster_ctarank() : 0u;
    // this CTA's share of the k-tiles and of the work items
    const int k_begin = kSplitK ? int(k_rank) * k_tiles / 2 : 0;
    const int k_end = kSplitK ? (int(k_rank) + 1) * k_tiles / 2 : k_tiles;
    const int first_item = kSplitK ? blockIdx.x >> 1 : blockIdx.x;
    const int item_step = kSplitK ? gridDim.x >> 1 : gridDim.x;
    const uint32_t b_base = a_base + C::kStages * C::kABytes;
    const uint32_t sfa_base = b_base + C::kStages * C::kBBytes;
    const uint32_t sfb_base = sfa_base + C::kStages * C::kSfaBytes;
    const uint32_t epi_base = sfb_base + C::kStages * C::kSfbBytes;
    const uint32_t bar_off = C::kStages * C::kStageBytes + C::kEpiBytes;
    Barriers* const bars = reinterpret_cast<Barriers*>(smem + bar_off);
    volatile uint32_t* const abort = &bars->abort;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&bars->full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&bars->sf_full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&bars->empty[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_init(ptx::smem_u32(&bars->acc_full[s]), (dual || ordered) ? 2 : 1);  // one commit per MMA issuer
            ptx::mbar_init(ptx::smem_u32(&bars->turn[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&bars->acc_empty[s]), kEpiWarps);
            ptx::mbar_init(ptx::smem_u32(&bars->overlap_free[s]), kEpiWarps);
        }
        for (int s = 0; s < C::kSfSets; ++s) ptx::mbar_init(ptx::smem_u32(&bars->sf_ready[s]), kSfWarps);
        if (kSplitK) ptx::mbar_init(ptx::smem_u32(&bars->recv_full), kEpiWarps);
        bars->abort = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tmap(&tm_a);
        ptx::prefetch_tmap(&tm_b);
        ptx::prefetch_tmap(&tm_d);
    }
    if (warp == 1) {
        ptx::tmem_alloc<1>(ptx::smem_u32(&bars->tmem_base), C::kTmemCols);
        ptx::tmem_relinquish<1>();
    }
    ptx::tc_fence_before();
    __syncthreads();
    // the other CTA's barriers exist before anyone signals across the pair
    if (kSplitK) ptx::cluster_sync();
    ptx::tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    // Everything above overlaps the tail of the previous kernel under a
    // programmatic launch; nothing below may run before its writes are visible.
    ptx::pdl_wait();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            WorkIter<BN> work(grp, M, N, tiles_m, tiles_n, first_item, item_step);
            Work wk;
            while (ok && work.next(wk)) {
                const int m0 = wk.a_row0;
                const int n0 = wk.b_row0;
                const uint8_t* const sfa_row = sfa + int64_t(m0 / kBM) * kq_dim * 512;
                const uint8_t* const sfb_row = sfb + int64_t(wk.sfb_tile) * kq_dim * 512;
                for (int kt = k_begin; kt < k_end; ++kt, ++it) {
                    const uint32_t s = it % kRing;
                    const uint32_t ph = (it / kRing) & 1u;
                    ok = wait_bar(ptx::smem_u32(&bars->empty[s]), ph ^ 1u, abort, kStatusProducer);
                    if (!ok) break;
                    const uint32_t full = ptx::smem_u32(&bars->full[s]);
                    const uint32_t sf_full = ptx::smem_u32(&bars->sf_full[s]);
                    // The scales have a barrier of their own: they are few bytes and land early,
                    // so the scale warps are done before the operand tiles arrive.
                    ptx::mbar_arrive_expect_tx(sf_full, C::kSfaBytes + C::kSfbBytes);
                    const int64_t koff = int64_t(kt) * C::kSfaBytes;
                    ptx::bulk_load(sfa_base + s * C::kSfaBytes, sfa_row + koff, C::kSfaBytes, sf_full);
#pragma unroll
                    for (int j = 0; j < C::kNAtoms; ++j) {
                        ptx::bulk_load(sfb_base + s * C::kSfbBytes + j * C::kSfaBytes,
                                       sfb_row + int64_t(j) * kq_dim * 512 + koff, C::kSfaBytes, sf_full);
                    }
                    // a short activation loads only its own rows (the A box is a_rows tall)
                    // packed e2m1 weights spread to one byte per value in shared memory, but the
                    // barrier counts the bytes read from global memory: half of the stage's B bytes
                    ptx::mbar_arrive_expect_tx(full, C::kABytes + C::kBBytes - (kBM - a_rows) * kBKBytes -
                                                         (KIND == 3 ? C::kBBytes / 2 : 0));
                    ptx::tma_load_2d(a_base + s * C::kABytes, &tm_a, kt * kBKBytes, m0, full);
                    ptx::tma_load_2d(b_base + s * C::kBBytes, &tm_b, kt * kBKBytes, n0, full);
                }
            }
            // let a dependent kernel start its prologue
            ptx::pdl_launch_dependents();
        }
    } else if (warp == 1 || warp == 10) {
        // ------------------------------------------------------------ MMA issuer(s)
        const int me = warp == 1 ? 0 : 1;
        if (lane == 0 && (me == 0 || dual || ordered)) {
            uint32_t it = 0;
            uint32_t t = 0;
            bool ok = true;
            WorkIter<BN> work(grp, M, N, tiles_m, tiles_n, first_item, item_step);
            Work wk;
            for (; ok && work.next(wk); ++t) {
                const uint32_t as = t & 1u;
                const uint32_t aph = (t >> 1) & 1u;
                // (with two issuers both wait here, also the one that has no k-tile in a tile of
                // one: its arrival below must not run ahead of the stage's previous use)
                ok = wait_bar(ptx::smem_u32(&bars->acc_empty[as]), aph ^ 1u, abort, kStatusMma);
                if (!ok) break;
                if (C::kOverlap != 0 && t > 0) {
                    // the previous tile's epilogue has drained the columns both stages share
                    ok = wait_bar(ptx::smem_u32(&bars->overlap_free[as ^ 1u]), ((t - 1) >> 1) & 1u,
                                  abort, kStatusMma);
                    if (!ok) break;
                }
                ptx::tc_fence_after();
                const uint32_t acc = tmem + ((me == 0 || ordered) ? as * C::kAccStride : C::kDualCol + as * BN);
                // a 64-wide tile uses half of a 128-row scale atom
                const uint32_t sfb_shift = BN == 64 ? uint32_t(wk.sfb_shift) : 0u;
                bool issued = false;
                for (int kt = k_begin; kt < k_end; ++kt, ++it) {
                    if (dual && ((kt - k_begin) & 1) != me) continue;
                    if (ordered && int(it & 1u) != me) continue;
                    const uint32_t s = it % kRing;
                    const uint32_t ph = (it / kRing) & 1u;
                    // the scales of this k-tile are in their set (the scale warps waited for the
                    // scale bytes); the stage's own barrier orders this thread after the TMA writes
                    ok = wait_bar(ptx::smem_u32(&bars->sf_ready[it % C::kSfSets]), (it / C::kSfSets) & 1u, abort,
                                  kStatusMma) &&
                         wait_bar(ptx::smem_u32(&bars->full[s]), ph, abort, kStatusMma);
                    // (in-order pair of issuers) the other thread has issued the MMAs of the previous k-iteration
                    if (ok && ordered && it > 0u) {
                        ok = wait_bar(ptx::smem_u32(&bars->turn[me]), ((it - 1u) >> 1) & 1u, abort, kStatusMma);
                    }
                    if (!ok) break;
                    ptx::tc_fence_after();
                    const uint32_t set = tmem + (it % C::kSfSets) * C::kSfCols;
                    const uint64_t adesc = ptx::smem_desc(a_base + s * C::kABytes, 16, 1024, 2);
                    const uint64_t bdesc = ptx::smem_desc(b_base + s * C::kBBytes, 16, 1024, 2);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        // 32 bytes of K per instruction: K = 32 (e4m3) or 64 (e2m1)
                        uint32_t atom, sf_id;
                        if constexpr (KIND == 0 || KIND == 3) {
                            atom = 0;
                            sf_id = k;
                        } else if constexpr (KIND == 1) {
                            atom = k;
                            sf_id = 0;
                        } else {
                            atom = k >> 1;
                            sf_id = (k & 1) * 2;
                        }
                        ptx::tc_mma_block_scaled<1, KIND>(
                            acc, adesc + uint64_t(k * 2), bdesc + uint64_t(k * 2),
                            instr_desc<BN, KIND>(sf_id), set + C::kSfaCol + atom * 4,
                            set + C::kSfbCol + atom * C::kNAtoms * 4 + sfb_shift,
                            (ordered ? (kt > k_begin || k > 0) : (issued || k > 0)) ? 1u : 0u);
                    }
                    issued = true;
                    if (ordered) {
                        // hand the turn over before the (slow) commit
                        ptx::tc_fence_before();
                        ptx::mbar_arrive(ptx::smem_u32(&bars->turn[me ^ 1]));
                    }
                    // stage s may be refilled once these MMAs have read it
                    ptx::tc_commit(ptx::smem_u32(&bars->empty[s]));
                }
                if (!ok) break;
                // a commit tracks the executing thread's operations: every issuer reports its own
                if (issued) {
                    ptx::tc_commit(ptx::smem_u32(&bars->acc_full[as]));
                } else {
                    ptx::mbar_arrive(ptx::smem_u32(&bars->acc_full[as]));
                }
            }
        }
    } else if (warp >= 2 + kEpiWarps) {
        // ------------------------------------------------------------ scales -> tensor memory (warps 6-9)
        // One SfAtom is 32 rows of 16 bytes; lane l of every lane quarter of tensor memory
        // holds row l in 4 columns (what tcgen05.cp.32x128b.warpx4 would write).  Each of
        // the four warps fills its own quarter from the same shared-memory image.
        const uint32_t quarter = (uint32_t(warp) & 3u) * 32u;
        uint32_t it = 0;
        bool ok = true;
        WorkIter<BN> work(grp, M, N, tiles_m, tiles_n, first_item, item_step);
        Work wk;
        while (ok && work.next(wk)) {
            for (int kt = k_begin; kt < k_end; ++kt, ++it) {
                const uint32_t s = it % kRing;
                ok = wait_bar(ptx::smem_u32(&bars->sf_full[s]), (it / kRing) & 1u, abort, kStatusProducer);
                if (ok && it >= uint32_t(C::kSfSets)) {
                    // the MMAs of k-tile it - kSfSets read this set: they are done once they
                    // have released their stage
                    const uint32_t prev = it - uint32_t(C::kSfSets);
                    ok = wait_bar(ptx::smem_u32(&bars->empty[prev % kRing]), (prev / kRing) & 1u, abort,
                                  kStatusProducer);
                }
                if (!ok) break;
                ptx::tc_fence_after();
                const uint32_t set = tmem + (quarter << 16) + (it % C::kSfSets) * C::kSfCols;
                const uint32_t src_a = sfa_base + s * C::kSfaBytes + uint32_t(lane) * 16u;
                const uint32_t src_b = sfb_base + s * C::kSfbBytes + uint32_t(lane) * 16u;
#pragma unroll
                for (int a = 0; a < C::kSfKAtoms; ++a) {
                    uint32_t r0, r1, r2, r3;
                    ptx::ld_shared_v4(src_a + a * 512, r0, r1, r2, r3);
                    ptx::tc_store_32x32_x4(set + C::kSfaCol + a * 4, r0, r1, r2, r3);
#pragma unroll
                    for (int j = 0; j < C::kNAtoms; ++j) {
                        ptx::ld_shared_v4(src_b + (j * C::kSfKAtoms + a) * 512, r0, r1, r2, r3);
                        ptx::tc_store_32x32_x4(set + C::kSfbCol + (a * C::kNAtoms + j) * 4, r0, r1, r2, r3);
                    }
                }
                ptx::tc_wait_st();
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars->sf_ready[it % C::kSfSets]));
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int ew = warp - 2;                  // staging buffer owner
        const uint32_t lane_base = (warp & 3) * 32;  // tensor-memory lanes this warp may read
        uint32_t t = 0;
        uint32_t stores = 0;
        bool ok = true;
        WorkIter<BN> work(grp, M, N, tiles_m, tiles_n, first_item, item_step);
        Work wk;
        const int ar = int(lane_base) + lane;  // accumulator row of this thread
        if (situ.sf != nullptr) zero_sf_padding(situ, (warp - 2) * 32 + lane);
        for (; ok && work.next(wk); ++t) {
            const int m0 = wk.out_row0;  // output row of accumulator row 0
            const int n0 = wk.out_col0;
            // this warp's 32 rows are all padding or all belong to a neighbouring group
            const bool warp_idle = int(lane_base) >= wk.row_hi || int(lane_base) + 32 <= wk.row_lo;
            const bool row_ok = ar >= wk.row_lo && ar < wk.row_hi;
            // whole tiles go out through TMA stores (a dense tail is clipped by the tensor map);
            // partial tiles are stored from registers, row by row, and so are tiles of at most
            // 32 rows (one warp, no staging round trip)
            const bool reg_store = direct_store != 0 || wk.row_lo != 0 || wk.row_hi <= 32 ||
                                   (wk.row_hi != kBM && grp.kind != kGroupDense);
            // per-tensor (dense) or per-group factor of the NVFP4 recipe
            const float scale = (KIND == 1 && alpha != nullptr) ? __ldg(alpha + wk.group) : 1.0f;
            const uint32_t as = t & 1u;
            const uint32_t aph = (t >> 1) & 1u;
            ok = wait_bar(ptx::smem_u32(&bars->acc_full[as]), aph, abort, kStatusEpilogue);
            if (!ok) break;
            ptx::tc_fence_after();
            const uint32_t acc = tmem + as * C::kAccStride + (lane_base << 16);
            if (KIND == 0 && epi_op == HQ_EPILOGUE_SITU_QUANT) {
                // quantising epilogue: 64 accumulator columns -> one group of 32 e4m3 outputs
                constexpr int kGroups = C::kChunks / 2;
#pragma unroll 1
                for (int gi = 0; gi < kGroups; ++gi) {
                    const int g = (C::kOverlap != 0 && as == 0) ? kGroups - 1 - gi : gi;
                    uint32_t r0[32], r1[32];
                    ptx::tc_load_32x32(acc + (2 * g) * kEpiChunk, r0);
                    ptx::tc_load_32x32(acc + (2 * g + 1) * kEpiChunk, r1);
                    ptx::tc_wait_ld();
                    if (C::kOverlap != 0 && gi == (C::kOverlapChunks - 1) / 2) {
                        ptx::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars->overlap_free[as]));
                    }
                    if (gi == kGroups - 1) {
                        ptx::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars->acc_empty[as]));
                    }
                    if (warp_idle) continue;
                    uint32_t y[16];
                    const __nv_bfloat16* const bc = bias != nullptr ? bias + n0 + 2 * g * kEpiChunk : nullptr;
                    situ_chunk(r0, bc, situ, &y[0]);
                    situ_chunk(r1, bc != nullptr ? bc + kEpiChunk : nullptr, situ, &y[8]);
                    uint4 lo, hi;
                    const uint32_t e = quant32_bf16(y, lo, hi);
                    const int64_t row = m0 + ar;
                    if (row_ok) {
                        const int kb = (n0 >> 6) + g;  // group of 32 output columns
                        uint4* const dst = reinterpret_cast<uint4*>(situ.q + row * situ.ldq + int64_t(kb) * 32);
                        dst[0] = lo;
                        dst[1] = hi;
                        situ.sf[((row >> 7) * (situ.kb_out >> 2) + (kb >> 2)) * 512 + (row & 31) * 16 +
                                ((row >> 5) & 3) * 4 + (kb & 3)] = uint8_t(e);
                    }
                }
                continue;
            }
            // Several chunks of columns shared with the other accumulator stage (FP4 kinds: the
            // scale sets take 48-96 columns): read them all into registers first, so that the
            // next tile's MMAs may start after three tensor-memory loads instead of after two
            // or three whole chunk iterations (convert, staging buffer, TMA store).
            constexpr int kPre = C::kOverlapChunks > 1 ? C::kOverlapChunks : 0;
            uint32_t ro[kPre > 0 ? kPre : 1][32];
            if constexpr (kPre > 0) {
#pragma unroll
                for (int j = 0; j < kPre; ++j) {
                    const int c = as == 0 ? C::kChunks - 1 - j : j;
                    ptx::tc_load_32x32(acc + c * kEpiChunk, ro[j]);
                }
                ptx::tc_wait_ld();
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars->overlap_free[as]));
            }
#pragma unroll 1
            for (int ci = 0; ci < C::kChunks; ++ci) {
                // stage 0 shares its highest columns with stage 1, stage 1 its lowest with stage 0
                const int c = (C::kOverlap != 0 && as == 0) ? C::kChunks - 1 - ci : ci;
                uint32_t r[32];
                if (kPre > 0 && ci < kPre) {
#pragma unroll
                    for (int j = 0; j < kPre; ++j) {
                        if (ci == j) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) r[i] = ro[j][i];
                        }
                    }
                } else {
                    ptx::tc_load_32x32(acc + c * kEpiChunk, r);
                    ptx::tc_wait_ld();
                }
                if constexpr (BN == 64 && !kSplitK) {
                    // the second issuer's accumulator (it has k-tiles whenever the tile has two or more)
                    if (dual && k_end - k_begin > 1) {
                        uint32_t r2[32];
                        ptx::tc_load_32x32(tmem + C::kDualCol + as * BN + (lane_base << 16) + c * kEpiChunk, r2);
                        ptx::tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(r2[i]));
                    }
                }
                if constexpr (kSplitK) {
                    // row `ar`, columns [32 c, 32 c + 32) of the 128 x 64 fp32 buffer
                    const uint32_t slot = recv_base + uint32_t(ar) * (BN * 4) + uint32_t(c) * (kEpiChunk * 4);
                    if (k_rank != 0) {
                        // an aborting CTA sends nothing more across the pair
                        if (*abort != 0u) {
                            ok = false;
                            break;
                        }
                        const uint32_t dst = ptx::mapa_cluster(slot, 0);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            ptx::st_cluster_v4(dst + j * 16, __uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                               __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                        }
                        if (ci == C::kChunks - 1) {
                            // every lane's stores are ordered before the warp's one remote arrive
                            __syncwarp();
                            if (lane == 0) {
                                ptx::mbar_arrive_cluster_addr(ptx::mapa_cluster(ptx::smem_u32(&bars->recv_full), 0));
                            }
                            ptx::tc_fence_before();
                            __syncwarp();
                            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars->acc_empty[as]));
                        }
                        continue;
                    }
                    if (ci == 0) {
                        // this tile's partial sums (one phase of the barrier per tile)
                        const uint64_t t0 = ptx::globaltimer_ns();
                        while (!ptx::mbar_try_wait_cluster(ptx::smem_u32(&bars->recv_full), t & 1u)) {
                            if (*abort != 0u || ptx::globaltimer_ns() - t0 > kTimeoutNs) {
                                *abort = 1u;
                                atomicOr(&g_status[0], uint32_t(kStatusEpilogue));
                                ok = false;
                                break;
                            }
                        }
                        if (!ok) break;
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float4 v;
                        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                     : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                                     : "r"(slot + j * 16));
                        r[4 * j] = __float_as_uint(__uint_as_float(r[4 * j]) + v.x);
                        r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + v.y);
                        r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + v.z);
                        r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + v.w);
                    }
                }
                if (C::kOverlap != 0 && kPre == 0 && ci == C::kOverlapChunks - 1) {
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars->overlap_free[as]));
                }
                if (ci == C::kChunks - 1) {
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars->acc_empty[as]));
                }
                uint32_t p[16];
                epilogue_chunk(r, p, scale, bias != nullptr ? bias + wk.bias_col0 + c * kEpiChunk : nullptr,
                               epi_op);
                const int row = m0 + ar;
                const int col = n0 + c * kEpiChunk;
                if (warp_idle) continue;
                if (epi_op == HQ_EPILOGUE_QUANT || epi_op == HQ_EPILOGUE_GATE_MUL_QUANT ||
                    epi_op == HQ_EPILOGUE_SIGMOID_GATE_MUL_QUANT) {
                    // The bf16 result (times the gate, as a bf16 product) re-quantised to MXFP8 per
                    // 32 columns: the reference's batch epilogues (csrc/kernel/gemm/epilogue.cuh:990-1051).
                    if (row_ok) {
                        if (epi_op != HQ_EPILOGUE_QUANT) {
                            const uint4* const gp =
                                reinterpret_cast<const uint4*>(situ.gate + int64_t(row) * situ.gate_ld + col);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const uint4 gq = __ldg(gp + j);
                                uint32_t gw[4] = {gq.x, gq.y, gq.z, gq.w};
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    if (epi_op == HQ_EPILOGUE_SIGMOID_GATE_MUL_QUANT) {
                                        const float lo = fmaf(0.5f, tanh_fast(0.5f * __uint_as_float(gw[i] << 16)), 0.5f);
                                        const float hi =
                                            fmaf(0.5f, tanh_fast(0.5f * __uint_as_float(gw[i] & 0xffff0000u)), 0.5f);
                                        const __nv_bfloat162 sg = __float22bfloat162_rn(make_float2(lo, hi));
                                        gw[i] = *reinterpret_cast<const uint32_t*>(&sg);
                                    }
                                    const __nv_bfloat162 prod =
                                        __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&p[4 * j + i]),
                                                *reinterpret_cast<const __nv_bfloat162*>(&gw[i]));
                                    p[4 * j + i] = *reinterpret_cast<const uint32_t*>(&prod);
                                }
                            }
                        }
                        uint4 lo, hi;
                        const uint32_t e = quant32_bf16(p, lo, hi);
                        const int kb = col >> 5;
                        uint4* const dst = reinterpret_cast<uint4*>(situ.q + int64_t(row) * situ.ldq + col);
                        dst[0] = lo;
                        dst[1] = hi;
                        situ.sf[(int64_t(row >> 7) * (situ.kb_out >> 2) + (kb >> 2)) * 512 + (row & 31) * 16 +
                                ((row >> 5) & 3) * 4 + (kb & 3)] = uint8_t(e);
                    }
                    continue;
                }
                if (reg_store) {
                    if (row_ok) {
                        uint4* dst = reinterpret_cast<uint4*>(out + int64_t(row) * ldo + col);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            dst[j] = make_uint4(p[4 * j], p[4 * j + 1], p[4 * j + 2], p[4 * j + 3]);
                        }
                    }
                } else {
                    const uint32_t buf =
                        epi_base + (ew * C::kEpiBufs + (stores % C::kEpiBufs)) * kEpiBufBytes;
                    // the TMA store that last read this buffer must be done with it
                    if (lane == 0) ptx::bulk_wait_read<C::kEpiBufs - 1>();
                    __syncwarp();
                    // 32 rows x 64 bytes, 64-byte swizzle: 16-byte chunk j of row r
                    // sits at chunk j ^ ((r >> 1) & 3)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t dst = buf + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst),
                                     "r"(p[4 * j]), "r"(p[4 * j + 1]), "r"(p[4 * j + 2]),
                                     "r"(p[4 * j + 3])
                                     : "memory");
                    }
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        ptx::tma_store_2d(&tm_d, buf, col, m0 + int(lane_base));
                        ptx::bulk_commit();
                    }
                    ++stores;
                }
            }
        }
        if (lane == 0) ptx::bulk_wait_read<0>();
    }

    if (*abort != 0u) {
        // bounded grace period for copies / MMAs still in flight before the
        // shared and tensor memory they target is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before();
    __syncthreads();
    // split-K: neither CTA of the pair leaves while the other may still store partial sums
    // into its shared memory or arrive on its barrier (every wait above is bounded, so both
    // get here)
    if (kSplitK) ptx::cluster_sync();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc<1>(tmem, C::kTmemCols);
    }
}

// Self-test of the bounded wait and of the way a timeout spreads: thread 0 waits, with a
// short limit, on a barrier that nothing ever arrives on; thread 32 waits on the same
// barrier with the ordinary limit and must leave as soon as it sees the abort flag thread
// 0 raises.  Nothing is in flight when the waits give up: no copies, no MMAs, no tensor
// memory.  What the host then reads through hq_device_status is what it would read after a
// GEMM role had timed out.
__global__ void __launch_bounds__(64, 1) wait_selftest_kernel(uint64_t limit_ns) {
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        ptx::mbar_init(ptx::smem_u32(&bar), 1);
        abort_flag = 0;
        ptx::fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        wait_bar(ptx::smem_u32(&bar), 0, &abort_flag, kStatusMma, limit_ns);
    } else if (threadIdx.x == 32) {
        // sees the flag within 32 polls of its being raised; its own limit never runs out
        if (wait_bar(ptx::smem_u32(&bar), 0, &abort_flag, kStatusEpilogue)) atomicOr(&g_status[0], 0x80u);
    }
    __syncwarp();
    __syncthreads();
}

// ---------------------------------------------------------------------------- M <= 16, plain scales
//
// Decode-sized GEMM whose block scales come in the plain row-major [rows, K / 32] layout
// (what the quantizer writes without the SfAtom swizzle), with the two fused forms of the
// reference's low-latency GEMM (csrc/kernel/gemm/low_latency_mma_gemm.cu:23-76): concat-K
// (a second input / weight pair accumulated into the same output) and dual output (a
// second weight multiplied by the same input).  128 x 64 tiles of the tcgen05 path; the
// 512-byte scale atoms the MMA wants are assembled in shared memory by a warp of 4-byte
// cp.async copies, one scale word per row and k-tile, that arrive on the stage's barrier.

struct LlParams {
    const uint8_t* sfa;   // [m, k1 / 32]
    const uint8_t* sfb;   // [n, k1 / 32]
    const uint8_t* sfa2;  // concat-K: [m, k2 / 32]
    const uint8_t* sfb2;  // concat-K: [n, k2 / 32]; dual output: [n2, k1 / 32]
    int64_t sfa_stride, sfb_stride, sfa2_stride, sfb2_stride;  // bytes between scale rows
    __nv_bfloat16* out;   // [m, n]
    __nv_bfloat16* out2;  // dual output: [m, n2]
    int64_t ldo, ldo2;
    int m, n, n2;            // n2 = 0 unless dual output
    int k_tiles1, k_tiles2;  // k_tiles2 = 0 unless concat-K
    int a_rows;              // rows of the A box (m rounded up to 8)
    int sigmoid;             // write sigmoid(bf16(result)) instead
};

// Warps: 0 loader, 1 MMA issuer 0, 2-5 epilogue, 6 scale builder, 7 scale copies, 8 MMA issuer 1.
// A stage holds 16 rows of A (the MMA reads 128 rows; what follows in shared memory only
// reaches accumulator rows that are never stored), so 16 stages fit; the scale copies and
// every second k-tile's MMAs have threads of their own.  Each of the two changes alone left
// the k-tile time where it was (one issuing thread needs about 640 cycles per k-tile; 8
// stages of loads that take about 5000 cycles to arrive allow one k-tile per 625 cycles).
constexpr int kLlThreads = 288;
constexpr int kLlStages = 16;
constexpr int kLlABytes = 16 * kBKBytes;
constexpr int kLlStageBytes = kLlABytes + 64 * kBKBytes + 512 + 512;
constexpr int kLlSmemBytes = kLlStages * kLlStageBytes + 1024 + 1024;
constexpr int kLlSfSets = 4;

__global__ void __launch_bounds__(kLlThreads, 1)
ll_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
               const __grid_constant__ CUtensorMap tm_a2, const __grid_constant__ CUtensorMap tm_b2,
               const LlParams p) {
    constexpr int BN = 64;
    using C = Cfg<BN, 0>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* const smem = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
    const uint32_t a_base = smem_base;
    const uint32_t b_base = a_base + kLlStages * kLlABytes;
    const uint32_t sfa_base = b_base + kLlStages * C::kBBytes;
    const uint32_t sfb_base = sfa_base + kLlStages * C::kSfaBytes;
    const uint32_t bar_off = kLlStages * kLlStageBytes;
    static_assert(kLlStages * 64 * kBKBytes >= (kBM - 16) * kBKBytes, "A over-read stays inside the B stages");
    static_assert(kLlStages <= int(sizeof(Barriers::full) / sizeof(uint64_t)), "one barrier pair per stage");
    static_assert(sizeof(Barriers) <= 1024, "barrier block");
    static_assert(C::kSfaCol + kLlSfSets * C::kSfCols <= C::kTmemCols, "scale sets fit the allocation");
    Barriers* const bars = reinterpret_cast<Barriers*>(smem + bar_off);
    volatile uint32_t* const abort = &bars->abort;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles1 = (p.n + BN - 1) / BN;
    const int num_tiles = tiles1 + (p.n2 + BN - 1) / BN;
    const int k_tiles = p.k_tiles1 + p.k_tiles2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kLlStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&bars->full[s]), 33);  // the loader + 32 scale-builder lanes
            ptx::mbar_init(ptx::smem_u32(&bars->empty[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_init(ptx::smem_u32(&bars->acc_full[s]), 2);  // one commit per MMA-issuing thread
            ptx::mbar_init(ptx::smem_u32(&bars->acc_empty[s]), kEpiWarps);
            ptx::mbar_init(ptx::smem_u32(&bars->turn[s]), 1);
        }
        for (int s = 0; s < kLlSfSets; ++s) ptx::mbar_init(ptx::smem_u32(&bars->sf_ready[s]), 1);
        bars->abort = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tmap(&tm_a);
        ptx::prefetch_tmap(&tm_b);
        ptx::prefetch_tmap(&tm_a2);
        ptx::prefetch_tmap(&tm_b2);
    }
    if (warp == 1) {
        ptx::tmem_alloc<1>(ptx::smem_u32(&bars->tmem_base), C::kTmemCols);
        ptx::tmem_relinquish<1>();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    ptx::pdl_wait();

    if (warp == 0) {
        // ------------------------------------------------------------ box loader
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                const bool second = tile >= tiles1;  // dual output: a tile of weight2
                const int n0 = (second ? tile - tiles1 : tile) * BN;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const uint32_t s = it % kLlStages;
                    ok = wait_bar(ptx::smem_u32(&bars->empty[s]), ((it / kLlStages) & 1u) ^ 1u, abort,
                                  kStatusProducer);
                    if (!ok) break;
                    const uint32_t full = ptx::smem_u32(&bars->full[s]);
                    ptx::mbar_arrive_expect_tx(full, p.a_rows * kBKBytes + C::kBBytes);
                    const bool tail = kt >= p.k_tiles1;  // concat-K: the second input / weight pair
                    const int x = (tail ? kt - p.k_tiles1 : kt) * kBKBytes;
                    ptx::tma_load_2d(a_base + s * kLlABytes, tail ? &tm_a2 : &tm_a, x, 0, full);
                    ptx::tma_load_2d(b_base + s * C::kBBytes, (tail || second) ? &tm_b2 : &tm_b, x, n0, full);
                }
            }
            ptx::pdl_launch_dependents();
        }
    } else if (warp == 6) {
        // ------------------------------------------------------------ scale builder
        // lane r writes the scale words of A row r and of B rows r and r + 32 where the
        // SfAtom has them: byte (row % 32) * 16 + (row / 32) * 4 of the stage's atom
        uint32_t it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
            const bool second = tile >= tiles1;
            const int n0 = (second ? tile - tiles1 : tile) * BN;
            const int n_rows = second ? p.n2 : p.n;
            for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                const uint32_t s = it % kLlStages;
                ok = wait_bar(ptx::smem_u32(&bars->empty[s]), ((it / kLlStages) & 1u) ^ 1u, abort, kStatusProducer);
                if (!ok) break;
                const bool tail = kt >= p.k_tiles1;
                const int64_t koff = int64_t(tail ? kt - p.k_tiles1 : kt) * 4;
                const uint8_t* const sa = tail ? p.sfa2 : p.sfa;
                const int64_t sa_stride = tail ? p.sfa2_stride : p.sfa_stride;
                const uint8_t* const sb = (tail || second) ? p.sfb2 : p.sfb;
                const int64_t sb_stride = (tail || second) ? p.sfb2_stride : p.sfb_stride;
                if (lane < p.m) ptx::cp_async_4(sfa_base + s * C::kSfaBytes + lane * 16, sa + lane * sa_stride + koff);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = n0 + lane + 32 * h;
                    if (row < n_rows) {
                        ptx::cp_async_4(sfb_base + s * C::kSfbBytes + lane * 16 + h * 4, sb + row * sb_stride + koff);
                    }
                }
                ptx::cp_async_arrive_noinc(ptx::smem_u32(&bars->full[s]));
            }
        }
    } else if (warp == 7) {
        // ------------------------------------------------------------ scale copies
        // shared memory -> tensor memory, into scale set it % kLlSfSets
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const uint32_t s = it % kLlStages;
                    ok = wait_bar(ptx::smem_u32(&bars->full[s]), (it / kLlStages) & 1u, abort, kStatusProducer);
                    if (!ok) break;
                    if (it >= uint32_t(kLlSfSets)) {
                        // the MMAs of k-tile it - kLlSfSets read this set: done once they released their stage
                        const uint32_t prev = it - uint32_t(kLlSfSets);
                        ok = wait_bar(ptx::smem_u32(&bars->empty[prev % kLlStages]), (prev / kLlStages) & 1u, abort,
                                      kStatusProducer);
                        if (!ok) break;
                    }
                    // the scale words were written by ordinary asynchronous copies; the
                    // tensor-memory copy reads them through the async proxy
                    ptx::fence_proxy_async_smem();
                    ptx::tc_fence_after();
                    const uint32_t set = tmem + (it % kLlSfSets) * C::kSfCols;
                    ptx::tc_copy_sf<1>(set + C::kSfaCol, ptx::smem_desc(sfa_base + s * C::kSfaBytes, 0, 128, 0));
                    ptx::tc_copy_sf<1>(set + C::kSfbCol, ptx::smem_desc(sfb_base + s * C::kSfbBytes, 0, 128, 0));
                    ptx::tc_commit(ptx::smem_u32(&bars->sf_ready[it % kLlSfSets]));
                }
            }
        }
    } else if (warp == 1 || warp == 8) {
        // ------------------------------------------------------------ MMA issuers
        // alternate k-tiles; after its MMAs a thread hands the turn to the other one (tcgen05
        // fences around an mbarrier arrive), so the MMAs reach the tensor core in k order
        if (lane == 0) {
            const uint32_t me = warp == 1 ? 0u : 1u;
            uint32_t it = 0;
            uint32_t t = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++t) {
                const uint32_t as = t & 1u;
                const uint32_t acc = tmem + as * C::kAccStride;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    if ((it & 1u) != me) continue;
                    const uint32_t s = it % kLlStages;
                    if (kt == 0) {
                        ok = wait_bar(ptx::smem_u32(&bars->acc_empty[as]), ((t >> 1) & 1u) ^ 1u, abort, kStatusMma);
                        if (!ok) break;
                    }
                    ok = wait_bar(ptx::smem_u32(&bars->sf_ready[it % kLlSfSets]), (it / kLlSfSets) & 1u, abort,
                                  kStatusMma) &&
                         wait_bar(ptx::smem_u32(&bars->full[s]), (it / kLlStages) & 1u, abort, kStatusMma);
                    if (ok && it > 0u) {
                        ok = wait_bar(ptx::smem_u32(&bars->turn[me]), ((it - 1u) >> 1) & 1u, abort, kStatusMma);
                    }
                    if (!ok) break;
                    ptx::tc_fence_after();
                    const uint32_t set = tmem + (it % kLlSfSets) * C::kSfCols;
                    const uint64_t adesc = ptx::smem_desc(a_base + s * kLlABytes, 16, 1024, 2);
                    const uint64_t bdesc = ptx::smem_desc(b_base + s * C::kBBytes, 16, 1024, 2);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        ptx::tc_mma_block_scaled<1, 0>(acc, adesc + uint64_t(k * 2), bdesc + uint64_t(k * 2),
                                                       instr_desc<BN, 0>(uint32_t(k)), set + C::kSfaCol,
                                                       set + C::kSfbCol, (kt > 0 || k > 0) ? 1u : 0u);
                    }
                    ptx::tc_fence_before();
                    ptx::mbar_arrive(ptx::smem_u32(&bars->turn[me ^ 1u]));
                    ptx::tc_commit(ptx::smem_u32(&bars->empty[s]));
                    // a commit tracks the executing thread's operations: each of the two threads
                    // commits the accumulator after its own last k-tile (K is a multiple of 256,
                    // so every tile has k-tiles of both)
                    if (kt >= k_tiles - 2) ptx::tc_commit(ptx::smem_u32(&bars->acc_full[as]));
                }
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------ epilogue
        const uint32_t lane_base = (warp & 3) * 32;
        uint32_t t = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++t) {
            const bool second = tile >= tiles1;
            const int n0 = (second ? tile - tiles1 : tile) * BN;
            const int n_rows = second ? p.n2 : p.n;
            __nv_bfloat16* const out = second ? p.out2 : p.out;
            const int64_t ldo = second ? p.ldo2 : p.ldo;
            const uint32_t as = t & 1u;
            ok = wait_bar(ptx::smem_u32(&bars->acc_full[as]), (t >> 1) & 1u, abort, kStatusEpilogue);
            if (!ok) break;
            ptx::tc_fence_after();
            if (lane_base == 0) {  // the only 32 accumulator rows that can hold one of the m <= 16 rows
                const uint32_t acc = tmem + as * C::kAccStride;
#pragma unroll 1
                for (int c = 0; c < BN / kEpiChunk; ++c) {
                    uint32_t r[32];
                    ptx::tc_load_32x32(acc + c * kEpiChunk, r);
                    ptx::tc_wait_ld();
                    if (lane < p.m) {
                        const int col = n0 + c * kEpiChunk;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t w[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                float lo = __uint_as_float(r[8 * j + 2 * i]);
                                float hi = __uint_as_float(r[8 * j + 2 * i + 1]);
                                if (p.sigmoid) {
                                    // sigmoid of the bfloat16 result, as a float computation
                                    lo = __bfloat162float(__float2bfloat16_rn(lo));
                                    hi = __bfloat162float(__float2bfloat16_rn(hi));
                                    lo = __fdiv_rn(1.0f, 1.0f + expf(-lo));
                                    hi = __fdiv_rn(1.0f, 1.0f + expf(-hi));
                                }
                                const __nv_bfloat162 v = __float22bfloat162_rn(make_float2(lo, hi));
                                w[i] = *reinterpret_cast<const uint32_t*>(&v);
                            }
                            // weight rows come in multiples of 8: whole 16-byte pieces
                            if (col + 8 * j < n_rows) {
                                *reinterpret_cast<uint4*>(out + int64_t(lane) * ldo + col + 8 * j) =
                                    make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        }
                    }
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars->acc_empty[as]));
        }
    }

    if (*abort != 0u) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc<1>(tmem, C::kTmemCols);
    }
}

// ---------------------------------------------------------------------------- 2-CTA tiles
//
// Pair kernel: a cluster of two CTAs computes one 256 x BN tile with
// tcgen05.mma.cta_group::2 (M = 256).  CTA r of the pair owns rows
// [128 r, 128 r + 128) of the A tile, rows [r BN/2, (r + 1) BN/2) of the B tile and the
// matching half of the accumulator; both CTAs hold the scales of all BN columns.
// Every CTA loads its own halves with plain (non-broadcast) TMA copies in the
// cta_group::2 form, which lets the bytes be counted on the leader's (rank 0)
// barrier; only the leader issues tcgen05.cp / tcgen05.mma.  It releases a stage with
// one tcgen05.commit to its own barrier, which its loader passes on to the other CTA,
// and publishes an accumulator with one commit per CTA.  The epilogue warps of
// both CTAs report to the leader's barriers.  Per CTA this halves the B traffic from
// L2 and leaves room for 6 stages instead of 4.

template <int BN, int KIND>
struct Cfg2 {
    static_assert(BN == 128 || BN == 256, "pair tile widths built");
    static constexpr int kABytes = kBM * kBKBytes;
    static constexpr int kBBytes = (BN / 2) * kBKBytes;
    static constexpr bool kFp8Kind = KIND == 0 || KIND == 3;  // mxf8f6f4: e4m3 x e4m3, or e4m3 x packed e2m1
    static constexpr int kSfKAtoms = kFp8Kind ? 1 : (KIND == 1 ? 4 : 2);
    static constexpr int kNAtoms = BN / 128;
    static constexpr int kSfaBytes = kSfKAtoms * 512;
    static constexpr int kSfbBytes = kNAtoms * kSfaBytes;
    static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
    // bytes a stage reads from global memory: packed e2m1 weights (KIND 3) are spread to one byte
    // per value by the copy, and the barrier counts what was read
    static constexpr int kStageTxBytes = kStageBytes - (KIND == 3 ? kBBytes / 2 : 0);
    static constexpr int kEpiBufs = 2;
    static constexpr int kEpiBytes = kEpiWarps * kEpiBufs * kEpiBufBytes;
    static constexpr int kBarBytes = 1024;
    static constexpr int kStagesFit = (kSmemBudget - kEpiBytes - kBarBytes - 1024) / kStageBytes;
    static constexpr int kStages = kStagesFit > 8 ? 8 : kStagesFit;
    static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + kBarBytes + 1024;
    // Scale columns of one k-iteration and how many such sets rotate in tensor memory.
    // The tcgen05.cp copies are issued by other warps than the MMAs: every asynchronous
    // instruction stalls the thread that issues it (measured per instruction: tcgen05.cp
    // 60-85 cycles, tcgen05.commit 88, a TMA copy 100-125) and those stalls only overlap
    // across warps.  One thread issuing 3 copies + 4 MMAs + 2 commits per k-tile spent 850
    // cycles on them; the MMAs alone take 512.  A set is free again once the MMAs that
    // read it have completed, so with 4 sets the copies run two k-tiles ahead.
    static constexpr int kSfCols = kSfKAtoms * 4 * (1 + kNAtoms);
    static constexpr int kSfSets = BN < 256 ? 4 : (kFp8Kind ? 4 : (KIND == 2 ? 3 : 2));
    // warps: 0 box loader, 1 MMA issuer, 2-5 epilogue, 6 scale loader, 7.. scale copies
    static constexpr int kCpWarps = kFp8Kind ? 1 : (KIND == 1 ? 3 : 2);
    // Two threads (warp 1 and the last warp) issue the MMAs of alternate k-tiles: issuing
    // 4 MMAs and the commit that releases the stage keeps one thread busy for longer
    // than the 512 cycles the MMAs run.  After its MMAs a thread
    // hands the turn to the other one (tcgen05 fences around an mbarrier arrive), so the
    // MMAs still reach the tensor core in k order.
    static constexpr int kThreads = 32 * (8 + kCpWarps);
    static constexpr int kSfRegion = kSfCols * kSfSets;
    static constexpr int kOverlap = BN == 256 ? (kSfRegion + 15) / 16 * 16 : 0;
    static constexpr int kAccStride = BN - kOverlap;
    static constexpr int kSfCol0 = kAccStride + BN;
    static constexpr int kColsUsed = kSfCol0 + kSfRegion;
    static constexpr int kTmemCols = kColsUsed <= 256 ? 256 : 512;
    static_assert(kColsUsed <= 512, "tensor memory budget");
    static constexpr int kChunks = BN / kEpiChunk;
    static constexpr int kOverlapChunks = (kOverlap + kEpiChunk - 1) / kEpiChunk;
    static_assert(kStages >= 2, "pipeline depth");
};

template <int BN, int KIND>
__device__ __forceinline__ uint32_t instr_desc_pair(uint32_t sf_id) {
    // (the fields and format codes of instr_desc; M = 256 across the pair)
    constexpr uint32_t fmt_a = (KIND == 0 || KIND == 3) ? 0u : 1u;
    constexpr uint32_t fmt_b = KIND == 0 ? 0u : (KIND == 3 ? 5u : 1u);
    constexpr uint32_t scale_fmt = KIND == 1 ? 0u : 1u;
    return (sf_id << 4) | (fmt_a << 7) | (fmt_b << 10) | (uint32_t(BN >> 3) << 17) | (scale_fmt << 23) |
           (uint32_t(256 >> 4) << 24) | (sf_id << 29);
}

// What one persistent-loop iteration of the 2-CTA kernel works on: a 256-row tile of the
// stacked A rows against BN rows of one weight.
struct PairWork {
    int a_row0;     // first of the tile's 256 stacked A rows (a multiple of 256)
    int b_row0;     // first of the BN weight rows in the stacked weights
    int row_lo;     // tile rows [row_lo, row_hi) belong to this item; the others are padding,
    int row_hi;     //   belong to another expert, or lie beyond M
    int out_row0;   // output row of tile row 0
    int out_col0;   // first output column
    int bias_col0;  // first bias element
};

// The grouped kinds on the 2-CTA tile (kGrouped; dense otherwise).  Batches and masked experts
// take it when their row count is a multiple of 256, so that no tile holds rows of two of
// them; an item is (expert, 256-row tile that holds valid rows of it, column tile).  The
// contiguous layout takes it when M is a multiple of 256: a tile whose four 64-row quarters
// belong to several experts is worked once per run of equal experts, each pass storing its own
// rows (the rule of the single-CTA kernel, with 256-row tiles).  The roles of the kernel walk
// the same sequence of items, each with its own copy of this iterator.
template <int BN, bool kGrouped>
struct PairWorkIter {
    GroupParams g;
    int M, N, tiles_m, tiles_n;
    int tile, stride;
    int pass = 0;        // contiguous: run of the current tile to work next
    int walk_group = 0;  // batch / masked: group of the last item and the number of
    int walk_base = 0;   //   (group, row tile) pairs before it

    __device__ PairWorkIter(const GroupParams& grp, int m, int n, int tm, int tn, int first, int step)
        : g(grp), M(m), N(n), tiles_m(tm), tiles_n(tn), tile(first), stride(step) {}

    __device__ bool next(PairWork& w) {
        if (!kGrouped || g.kind == kGroupContiguous) {
            if (tile >= tiles_m * tiles_n) return false;
            const TileCoord tc = tile_coord(tile, tiles_m, tiles_n);
            w.a_row0 = tc.m * 256;
            w.out_row0 = w.a_row0;
            w.out_col0 = tc.n * BN;
            w.row_lo = 0;
            w.row_hi = min(256, M - w.a_row0);
            int group = 0;
            bool last = true;
            if constexpr (kGrouped) {
                int e[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int row = w.a_row0 + 64 * q;
                    e[q] = row < M ? min(max(__ldg(g.table + row), 0), g.count - 1) : e[q > 0 ? q - 1 : 0];
                }
                int start = 0, run = 0, cur = e[0];
                bool found = false;
                group = e[0];
#pragma unroll
                for (int q = 1; q <= 4; ++q) {
                    const bool ends = q == 4 || e[q & 3] != e[q - 1];  // the run [start, q) of quarters ends here
                    if (!found && ends) {
                        if (run == pass) {
                            w.row_lo = 64 * start;
                            w.row_hi = min(64 * q, M - w.a_row0);
                            group = cur;
                            last = q == 4;
                            found = true;
                        } else {
                            ++run;
                            start = q;
                            cur = e[q & 3];
                        }
                    }
                }
                pass = last ? 0 : pass + 1;
            }
            w.b_row0 = group * N + tc.n * BN;
            w.bias_col0 = w.b_row0;
            if (last) tile += stride;
            return true;
        }
        // batch / masked
        const int pair = tile / tiles_n;
        const int nt = tile - pair * tiles_n;
        int first, valid;
        for (;;) {
            if (walk_group >= g.count) return false;
            first = walk_group * g.rows;
            valid = g.kind == kGroupMasked ? min(max(__ldg(g.table + walk_group), 0), g.rows) : g.rows;
            const int cnt = (valid + 255) / 256;
            if (pair < walk_base + cnt) break;
            walk_base += cnt;
            ++walk_group;
        }
        const int rt = pair - walk_base;
        w.a_row0 = first + rt * 256;
        w.row_lo = 0;
        w.row_hi = min(256, valid - rt * 256);
        w.b_row0 = walk_group * N + nt * BN;
        w.bias_col0 = w.b_row0;
        if (g.kind == kGroupBatch) {
            w.out_row0 = w.a_row0 - first;
            w.out_col0 = w.b_row0;
        } else {
            w.out_row0 = w.a_row0;
            w.out_col0 = nt * BN;
        }
        tile += stride;
        return true;
    }
};

// What the grouped 2-CTA kernel needs beyond the tensor maps: the groups, and the output for
// the rows it stores from registers (tiles that are only partly this item's).
struct PairGroupArgs {
    GroupParams grp;
    __nv_bfloat16* out;
    int64_t ldo;
    int m;  // stacked A rows
    int n;  // columns per weight
};

// Column-parallel all-gather fused into the epilogue (kGather): besides its own output, a rank
// stores every finished chunk of a tile into the same columns of its peers' outputs (symmetric
// memory mapped over NVLink): the TMA store that writes the staged chunk to the local output
// is repeated with a tensor map over each peer's matrix.  Every LOAD of the kernel (operands,
// scales) is from this GPU's memory.
template <bool kGather>
struct GatherMaps {
    int count;
};
template <>
struct GatherMaps<true> {
    CUtensorMap out[7];  // the peers' outputs, each map starting at this rank's first column
    int count;
};

template <int BN, int KIND, bool kGather = false, bool kGrouped = false>
__global__ void __launch_bounds__((Cfg2<BN, KIND>::kThreads), 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ CUtensorMap tm_d, const __grid_constant__ CUtensorMap tm_sfa,
                 const __grid_constant__ CUtensorMap tm_sfb, const float* __restrict__ alpha,
                 const __nv_bfloat16* __restrict__ bias, int epi_op, int k_tiles, int kq_dim, int tiles_m,
                 int tiles_n, const __grid_constant__ GatherMaps<kGather> peers, const PairGroupArgs ga) {
    using C = Cfg2<BN, KIND>;
    using Iter = PairWorkIter<BN, kGrouped>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* const smem = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
    const uint32_t a_base = smem_base;
    const uint32_t b_base = a_base + C::kStages * C::kABytes;
    const uint32_t sfa_base = b_base + C::kStages * C::kBBytes;
    const uint32_t sfb_base = sfa_base + C::kStages * C::kSfaBytes;
    const uint32_t epi_base = sfb_base + C::kStages * C::kSfbBytes;
    const uint32_t bar_off = C::kStages * C::kStageBytes + C::kEpiBytes;
    Barriers* const bars = reinterpret_cast<Barriers*>(smem + bar_off);
    volatile uint32_t* const abort = &bars->abort;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();  // 0 = leader
    const bool leader = rank == 0;
    const int cluster_id = blockIdx.x >> 1;
    const int num_clusters = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            // the leader's copy collects the bytes of both CTAs after one
            // expect_tx arrival of the leader's producer
            ptx::mbar_init(ptx::smem_u32(&bars->full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&bars->empty[s]), 1);  // one tcgen05.commit
        }
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_init(ptx::smem_u32(&bars->acc_full[s]), 2);  // one commit per MMA-issuing thread
            ptx::mbar_init(ptx::smem_u32(&bars->acc_empty[s]), 2 * kEpiWarps);  // leader's copy is used
            ptx::mbar_init(ptx::smem_u32(&bars->overlap_free[s]), 2 * kEpiWarps);
        }
        for (int s = 0; s < C::kSfSets; ++s) ptx::mbar_init(ptx::smem_u32(&bars->sf_ready[s]), C::kCpWarps);
        for (int s = 0; s < 2; ++s) ptx::mbar_init(ptx::smem_u32(&bars->turn[s]), 1);
        bars->abort = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tmap(&tm_a);
        ptx::prefetch_tmap(&tm_b);
        ptx::prefetch_tmap(&tm_d);
        ptx::prefetch_tmap(&tm_sfa);
        ptx::prefetch_tmap(&tm_sfb);
    }
    if (warp == 1) {
        ptx::tmem_alloc<2>(ptx::smem_u32(&bars->tmem_base), C::kTmemCols);
        ptx::tmem_relinquish<2>();
    }
    ptx::tc_fence_before();
    __syncthreads();
    // barriers of both CTAs are initialised before anyone signals across the pair
    ptx::cluster_sync();
    ptx::tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    ptx::pdl_wait();

    if (warp == 0) {
        // ------------------------------------------------------------ box loader (both CTAs)
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            Iter walk(ga.grp, ga.m, ga.n, tiles_m, tiles_n, cluster_id, num_clusters);
            PairWork wk;
            while (ok && walk.next(wk)) {
                const int m0 = wk.a_row0 + int(rank) * kBM;
                const int n0 = wk.b_row0 + int(rank) * (BN / 2);
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const uint32_t s = it % C::kStages;
                    ok = wait_bar(ptx::smem_u32(&bars->empty[s]), ((it / C::kStages) & 1u) ^ 1u, abort,
                                  kStatusProducer);
                    if (!ok) break;
                    // The MMA threads release a stage with one commit, to the leader's barrier; the
                    // leader's loader passes it on.  A second commit costs the issuing thread about
                    // 300 cycles per k-tile, this relaxed arrival about 200 on a thread with slack
                    // (what it reports, the MMAs' reads of the stage, completed before the commit).
                    if (leader && it >= uint32_t(C::kStages)) {
                        ptx::mbar_arrive_cluster_relaxed(ptx::mapa_cluster(ptx::smem_u32(&bars->empty[s]), 1));
                    }
                    const uint32_t full = ptx::mapa_cluster(ptx::smem_u32(&bars->full[s]), 0);
                    // Bytes of all four loader threads of the pair are counted on the leader's
                    // barrier; only this thread registers them (the count may go negative in
                    // between).
                    if (leader) ptx::mbar_arrive_expect_tx(ptx::smem_u32(&bars->full[s]), 2 * C::kStageTxBytes);
                    ptx::tma_load_2d_pair(a_base + s * C::kABytes, &tm_a, kt * kBKBytes, m0, full);
                    ptx::tma_load_2d_pair(b_base + s * C::kBBytes, &tm_b, kt * kBKBytes, n0, full);
                }
            }
            ptx::pdl_launch_dependents();
        }
    } else if (warp == 6) {
        // ------------------------------------------------------------ scale loader (both CTAs)
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            Iter walk(ga.grp, ga.m, ga.n, tiles_m, tiles_n, cluster_id, num_clusters);
            PairWork wk;
            while (ok && walk.next(wk)) {
                const int sfa_atom_row = (wk.a_row0 / 128 + int(rank)) * kq_dim;
                const int sfb_atom_row = (wk.b_row0 / 128) * kq_dim;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const uint32_t s = it % C::kStages;
                    ok = wait_bar(ptx::smem_u32(&bars->empty[s]), ((it / C::kStages) & 1u) ^ 1u, abort,
                                  kStatusProducer);
                    if (!ok) break;
                    const uint32_t full = ptx::mapa_cluster(ptx::smem_u32(&bars->full[s]), 0);
                    // scale atoms are rows of 128 32-bit words
                    ptx::tma_load_2d_pair(sfa_base + s * C::kSfaBytes, &tm_sfa, 0,
                                          sfa_atom_row + kt * C::kSfKAtoms, full);
#pragma unroll
                    for (int j = 0; j < C::kNAtoms; ++j) {
                        ptx::tma_load_2d_pair(sfb_base + s * C::kSfbBytes + j * C::kSfaBytes, &tm_sfb, 0,
                                              sfb_atom_row + j * kq_dim + kt * C::kSfKAtoms, full);
                    }
                }
            }
        }
    } else if (warp >= 7 && warp < 7 + C::kCpWarps) {
        // ------------------------------------------------------------ scale copies (leader only)
        // shared memory -> tensor memory of both CTAs, into scale set it % kSfSets
        if (leader && lane == 0) {
            const int cw = warp - 7;
            bool ok = true;
            Iter walk(ga.grp, ga.m, ga.n, tiles_m, tiles_n, cluster_id, num_clusters);
            PairWork wk;
            uint32_t total_its = 0;
            for (uint32_t it = 0; ok; ++it) {
                if (it == total_its) {  // the k-tiles of the next item
                    if (!walk.next(wk)) break;
                    total_its += uint32_t(k_tiles);
                }
                const uint32_t s = it % C::kStages;
                ok = wait_bar(ptx::smem_u32(&bars->full[s]), (it / C::kStages) & 1u, abort, kStatusProducer);
                if (!ok) break;
                if (it >= uint32_t(C::kSfSets)) {
                    // the MMAs of k-tile it - kSfSets read this set: they are done once they
                    // have released their stage
                    const uint32_t prev = it - uint32_t(C::kSfSets);
                    ok = wait_bar(ptx::smem_u32(&bars->empty[prev % C::kStages]), (prev / C::kStages) & 1u, abort,
                                  kStatusProducer);
                    if (!ok) break;
                }
                ptx::tc_fence_after();
                const uint32_t set = tmem + C::kSfCol0 + (it % C::kSfSets) * C::kSfCols;
#pragma unroll
                for (int a = 0; a < C::kSfKAtoms; ++a) {
                    if ((a * (1 + C::kNAtoms)) % C::kCpWarps == cw) {
                        ptx::tc_copy_sf<2>(set + a * 4,
                                           ptx::smem_desc(sfa_base + s * C::kSfaBytes + a * 512, 0, 128, 0));
                    }
#pragma unroll
                    for (int j2 = 0; j2 < C::kNAtoms; ++j2) {
                        if ((a * (1 + C::kNAtoms) + 1 + j2) % C::kCpWarps == cw) {
                            ptx::tc_copy_sf<2>(
                                set + C::kSfKAtoms * 4 + (a * C::kNAtoms + j2) * 4,
                                ptx::smem_desc(sfb_base + s * C::kSfbBytes + (j2 * C::kSfKAtoms + a) * 512, 0, 128,
                                               0));
                        }
                    }
                }
                ptx::tc_commit_pair(ptx::mapa_cluster(ptx::smem_u32(&bars->sf_ready[it % C::kSfSets]), 0));
            }
        }
    } else if (warp == 1 || warp == 7 + C::kCpWarps) {
        // ------------------------------------------------------------ MMA issuers (leader only)
        if (leader && lane == 0) {
            const uint32_t me = warp == 1 ? 0u : 1u;  // this thread issues the k-iterations it & 1 == me
            uint32_t it = 0;
            uint32_t t = 0;
            bool ok = true;
            Iter walk(ga.grp, ga.m, ga.n, tiles_m, tiles_n, cluster_id, num_clusters);
            PairWork wk;
            for (; ok && walk.next(wk); ++t) {
                const uint32_t as = t & 1u;
                const uint32_t aph = (t >> 1) & 1u;
                const uint32_t acc = tmem + as * C::kAccStride;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    if ((it & 1u) != me) {
                        if (k_tiles == 1) {
                            // A tile of one k-tile has nothing for this thread, but the accumulator's
                            // barrier expects both threads.  The arrival may not run ahead of the
                            // previous use of this accumulator stage, hence the same wait the
                            // issuing thread makes.
                            ok = wait_bar(ptx::smem_u32(&bars->acc_empty[as]), aph ^ 1u, abort, kStatusMma);
                            if (!ok) break;
                            const uint32_t accf = ptx::smem_u32(&bars->acc_full[as]);
                            ptx::mbar_arrive(accf);
                            ptx::mbar_arrive_cluster_relaxed(ptx::mapa_cluster(accf, 1));
                        }
                        continue;
                    }
                    const uint32_t s = it % C::kStages;
                    if (kt == 0) {
                        // first k-tile of a tile: the accumulator stage must have been drained
                        ok = wait_bar(ptx::smem_u32(&bars->acc_empty[as]), aph ^ 1u, abort, kStatusMma);
                        if (ok && C::kOverlap != 0 && t > 0) {
                            ok = wait_bar(ptx::smem_u32(&bars->overlap_free[as ^ 1u]), ((t - 1) >> 1) & 1u, abort,
                                          kStatusMma);
                        }
                        if (!ok) break;
                    }
                    // The scale copies of this k-tile have landed.  Every copy warp waited for the
                    // stage's barrier before it copied and committed, so the operand boxes of both
                    // CTAs have landed too: no second wait here (each one costs this thread, which
                    // sets the pace, 50-100 cycles).
                    ok = wait_bar(ptx::smem_u32(&bars->sf_ready[it % C::kSfSets]), (it / C::kSfSets) & 1u, abort,
                                  kStatusMma);
                    // the other thread has issued the MMAs of the previous k-iteration
                    if (ok && it > 0u) {
                        ok = wait_bar(ptx::smem_u32(&bars->turn[me]), ((it - 1u) >> 1) & 1u, abort, kStatusMma);
                    }
                    if (!ok) break;
                    ptx::tc_fence_after();
                    const uint32_t set = tmem + C::kSfCol0 + (it % C::kSfSets) * C::kSfCols;
                    const uint64_t adesc = ptx::smem_desc(a_base + s * C::kABytes, 16, 1024, 2);
                    const uint64_t bdesc = ptx::smem_desc(b_base + s * C::kBBytes, 16, 1024, 2);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        uint32_t atom, sf_id;
                        if constexpr (KIND == 0 || KIND == 3) {
                            atom = 0;
                            sf_id = k;
                        } else if constexpr (KIND == 1) {
                            atom = k;
                            sf_id = 0;
                        } else {
                            atom = k >> 1;
                            sf_id = (k & 1) * 2;
                        }
                        ptx::tc_mma_block_scaled<2, KIND>(
                            acc, adesc + uint64_t(k * 2), bdesc + uint64_t(k * 2),
                            instr_desc_pair<BN, KIND>(sf_id), set + atom * 4,
                            set + C::kSfKAtoms * 4 + atom * C::kNAtoms * 4, (kt > 0 || k > 0) ? 1u : 0u);
                    }
                    // hand the turn over before the (slow) commits
                    ptx::tc_fence_before();
                    ptx::mbar_arrive(ptx::smem_u32(&bars->turn[me ^ 1u]));
                    // the loaders of both CTAs may refill stage s once these MMAs have read it
                    // (the leader's loader passes the release on to the other CTA)
                    ptx::tc_commit_pair(ptx::mapa_cluster(ptx::smem_u32(&bars->empty[s]), 0));
                    // A commit tracks the operations of the thread that executes it, so each of
                    // the two threads commits the accumulator after its own last k-tile of the
                    // tile; the epilogue starts when both have completed.
                    if (kt >= k_tiles - 2) {
                        const uint32_t accf = ptx::smem_u32(&bars->acc_full[as]);
                        ptx::tc_commit_pair(ptx::mapa_cluster(accf, 0));
                        ptx::tc_commit_pair(ptx::mapa_cluster(accf, 1));
                    }
                }
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------ epilogue (both CTAs)
        const int ew = warp - 2;
        const uint32_t lane_base = (warp & 3) * 32;
        const float scale = (KIND == 1 && alpha != nullptr) ? __ldg(alpha) : 1.0f;
        uint32_t t = 0;
        uint32_t stores = 0;
        bool ok = true;
        Iter walk(ga.grp, ga.m, ga.n, tiles_m, tiles_n, cluster_id, num_clusters);
        PairWork wk;
        for (; ok && walk.next(wk); ++t) {
            const int m0 = wk.out_row0 + int(rank) * kBM;
            const int n0 = wk.out_col0;
            // rows of this CTA's half of the tile that belong to the item
            const int half_lo = min(max(wk.row_lo - int(rank) * kBM, 0), kBM);
            const int half_hi = min(max(wk.row_hi - int(rank) * kBM, 0), kBM);
            // (a dense tile that sticks out beyond M is clipped by the TMA store; the grouped kinds
            // come here with whole tiles inside M only)
            const bool partial = kGrouped && (half_lo != 0 || half_hi != kBM);
            const uint32_t as = t & 1u;
            const uint32_t aph = (t >> 1) & 1u;
            ok = wait_bar(ptx::smem_u32(&bars->acc_full[as]), aph, abort, kStatusEpilogue);
            if (!ok) break;
            ptx::tc_fence_after();
            const uint32_t acc = tmem + as * C::kAccStride + (lane_base << 16);
            // chunks shared with the other accumulator stage are read into registers first (as
            // in the single-CTA kernel), so that the next tile's MMAs may start early
            constexpr int kPre = C::kOverlapChunks > 1 ? C::kOverlapChunks : 0;
            uint32_t ro[kPre > 0 ? kPre : 1][32];
            if constexpr (kPre > 0) {
#pragma unroll
                for (int j = 0; j < kPre; ++j) {
                    const int c = as == 0 ? C::kChunks - 1 - j : j;
                    ptx::tc_load_32x32(acc + c * kEpiChunk, ro[j]);
                }
                ptx::tc_wait_ld();
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive_cluster_relaxed(ptx::mapa_cluster(ptx::smem_u32(&bars->overlap_free[as]), 0));
                }
            }
#pragma unroll 1
            for (int ci = 0; ci < C::kChunks; ++ci) {
                const int c = (C::kOverlap != 0 && as == 0) ? C::kChunks - 1 - ci : ci;
                uint32_t r[32];
                if (kPre > 0 && ci < kPre) {
#pragma unroll
                    for (int j = 0; j < kPre; ++j) {
                        if (ci == j) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) r[i] = ro[j][i];
                        }
                    }
                } else {
                    ptx::tc_load_32x32(acc + c * kEpiChunk, r);
                    ptx::tc_wait_ld();
                }
                // The arrivals below tell the leader's MMA threads that tensor-memory reads have
                // completed (tcgen05.wait::ld); no shared or global data rides on them.
                if (C::kOverlap != 0 && kPre == 0 && ci == C::kOverlapChunks - 1) {
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        ptx::mbar_arrive_cluster_relaxed(ptx::mapa_cluster(ptx::smem_u32(&bars->overlap_free[as]), 0));
                    }
                }
                if (ci == C::kChunks - 1) {
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        ptx::mbar_arrive_cluster_relaxed(ptx::mapa_cluster(ptx::smem_u32(&bars->acc_empty[as]), 0));
                    }
                }
                uint32_t p[16];
                epilogue_chunk(r, p, scale, bias != nullptr ? bias + wk.bias_col0 + c * kEpiChunk : nullptr, epi_op);
                if constexpr (kGrouped) {
                    if (partial) {
                        // only some rows of this half belong to the item: each thread stores its
                        // own row's 32 columns from registers, or nothing
                        const int r_half = int(lane_base) + lane;
                        if (r_half >= half_lo && r_half < half_hi) {
                            uint4* const dst = reinterpret_cast<uint4*>(ga.out + int64_t(m0 + r_half) * ga.ldo + n0 +
                                                                        c * kEpiChunk);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                dst[j] = make_uint4(p[4 * j], p[4 * j + 1], p[4 * j + 2], p[4 * j + 3]);
                            }
                        }
                        continue;
                    }
                }
                if constexpr (kGather) {
                    // Two neighbouring chunks are staged as ONE box of 32 rows x 128 bytes (the warp's
                    // two buffers, 128-byte swizzle) and stored together: rows of 128 bytes use
                    // NVLink better than rows of 64 (measured on 4 GPUs).  Chunks come in ascending
                    // or descending order, so chunk c's partner c ^ 1 is always the next or the previous one.
                    const uint32_t buf = epi_base + ew * C::kEpiBufs * kEpiBufBytes;
                    if ((ci & 1) == 0) {
                        if (lane == 0) ptx::bulk_wait_read<0>();
                        __syncwarp();
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t piece = uint32_t((c & 1) * 4 + j);
                        const uint32_t dst = buf + lane * 128 + ((piece ^ (lane & 7)) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(p[4 * j]),
                                     "r"(p[4 * j + 1]), "r"(p[4 * j + 2]), "r"(p[4 * j + 3])
                                     : "memory");
                    }
                    if ((ci & 1) != 0) {
                        ptx::fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            const int col = n0 + (c & ~1) * kEpiChunk;
                            ptx::tma_store_2d(&tm_d, buf, col, m0 + int(lane_base));
                            for (int q = 0; q < peers.count; ++q) {
                                ptx::tma_store_2d(&peers.out[q], buf, col, m0 + int(lane_base));
                            }
                            ptx::bulk_commit();
                        }
                    }
                    continue;
                }
                const uint32_t buf = epi_base + (ew * C::kEpiBufs + (stores % C::kEpiBufs)) * kEpiBufBytes;
                if (lane == 0) ptx::bulk_wait_read<C::kEpiBufs - 1>();
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t dst = buf + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(p[4 * j]),
                                 "r"(p[4 * j + 1]), "r"(p[4 * j + 2]), "r"(p[4 * j + 3])
                                 : "memory");
                }
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    ptx::tma_store_2d(&tm_d, buf, n0 + c * kEpiChunk, m0 + int(lane_base));
                    ptx::bulk_commit();
                }
                ++stores;
            }
        }
        if constexpr (kGather) {
            // the stores into the peers' memory have been performed, not only read from shared
            // memory, before the kernel is seen as complete
            if (lane == 0) {
                ptx::bulk_wait<0>();
                __threadfence_system();
            }
        } else {
            if (lane == 0) ptx::bulk_wait_read<0>();
        }
    }

    if (*abort != 0u) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before();
    __syncthreads();
    // neither CTA may leave while the other can still signal its barriers or
    // while MMAs of the pair read its shared memory
    ptx::cluster_sync();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc<2>(tmem, C::kTmemCols);
    }
}

// ---------------------------------------------------------------------------- small M
#include "decode.cuh"

// ---------------------------------------------------------------------------- host

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            p = nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// rank-2 row-major tensor map: `inner` elements per row, `rows` rows, `pitch` bytes between rows
bool make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, uint64_t inner,
                  uint64_t rows, uint64_t pitch, uint32_t box_inner, uint32_t box_rows,
                  CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {inner, rows};
    const cuuint64_t strides[1] = {pitch};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Per-device, once: the opt-in to more than 48 KB of dynamic shared memory for one kernel.
// A failed attempt is not remembered, so the next call tries (and reports) again.
struct SmemOptIn {
    std::mutex mu;
    bool done[64] = {};
    template <typename Kernel>
    cudaError_t ensure(Kernel kernel, int bytes, int* dev_out = nullptr) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (dev_out != nullptr) *dev_out = dev;
        std::lock_guard<std::mutex> lock(mu);
        if (dev >= 0 && dev < 64 && done[dev]) return cudaSuccess;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e == cudaSuccess && dev >= 0 && dev < 64) done[dev] = true;
        return e;
    }
};

struct GemmArgs {
    const void* a;
    const void* b;
    const uint8_t* sfa;
    const uint8_t* sfb;
    const float* alpha;
    const __nv_bfloat16* bias;
    int epi_op;
    SituParams situ;
    __nv_bfloat16* out;
    int64_t ldo;
    int m, n;          // rows of A (all groups stacked) and columns per weight
    GroupParams grp;
    int64_t k_bytes;
    int kq_dim;
    int sm_count;
    bool pdl;
    bool early_weights = false;  // with pdl: b and sfb may be read before the preceding kernel completes
    bool direct_store;
    cudaStream_t stream;
};

// Split-K is taken for a dense problem with one row of at most sm_count / 2 64-wide tiles and
// at least 8 k-tiles (HALOPS_B200_SPLITK=0 turns it off; read on every call).
bool split_k_chosen(int group_kind, int tiles_m, int tiles_n, int k_tiles, int sm_count, int epi_op) {
    const char* e = getenv("HALOPS_B200_SPLITK");
    if (e != nullptr && e[0] == '0') return false;
    return group_kind == kGroupDense && tiles_m == 1 && 2 * tiles_n <= sm_count && k_tiles >= 8 &&
           (epi_op == HQ_EPILOGUE_IDENTITY || epi_op == HQ_EPILOGUE_SIGMOID);
}

// 2: the single-CTA kernel issues its MMAs from two threads in k order (see the kernel);
// 0 with HALOPS_B200_ISSUERS=1 (read on every call)
int issuers_in_order() {
    const char* e = getenv("HALOPS_B200_ISSUERS");
    return e != nullptr && e[0] == '1' ? 0 : 2;
}

template <int BN, int KIND>
int launch_tile(const GemmArgs& g, char* err, size_t errlen) {
    using C = Cfg<BN, KIND>;
    static SmemOptIn opt_in;
    HQ_CUDA_TRY(opt_in.ensure(gemm_kernel<BN, KIND>, C::kSmemBytes));

    CUtensorMap tm_a, tm_b, tm_d;
    // M < 128: the A box holds only the rows that exist (rounded up to the 8-row
    // swizzle period); the other rows of the shared-memory tile keep stale bytes,
    // which only feed accumulator rows that are never stored
    const int64_t rows_a = g.m;
    const int64_t rows_b = int64_t(g.grp.kind == kGroupDense ? 1 : g.grp.count) * g.n;
    // output: [rows, count * N] for batches, else [M, N]
    const int64_t out_rows = g.grp.kind == kGroupBatch ? g.grp.rows : g.m;
    const int64_t out_cols = g.grp.kind == kGroupBatch ? rows_b : g.n;
    const int a_rows = rows_a >= kBM ? kBM : int((rows_a + 7) / 8 * 8);
    const bool maps_ok =
        make_tmap_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, g.a, uint64_t(g.k_bytes), uint64_t(rows_a),
                     uint64_t(g.k_bytes), kBKBytes, uint32_t(a_rows), CU_TENSOR_MAP_SWIZZLE_128B) &&
        // KIND 3: packed e2m1 weights; the copy spreads every 16 values (8 bytes) over 16 bytes
        // of shared memory, the form the mxf8f6f4 MMA reads 4-bit operands in, so a box of
        // 128 values per row fills the same 128 bytes as 128 e4m3 values
        (KIND == 3 ? make_tmap_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, g.b, uint64_t(g.k_bytes),
                                  uint64_t(rows_b), uint64_t(g.k_bytes / 2), kBKBytes, BN,
                                  CU_TENSOR_MAP_SWIZZLE_128B)
                   : make_tmap_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, g.b, uint64_t(g.k_bytes), uint64_t(rows_b),
                                  uint64_t(g.k_bytes), kBKBytes, BN, CU_TENSOR_MAP_SWIZZLE_128B)) &&
        // (the quantising epilogue stores from registers; its map only has to be valid)
        make_tmap_2d(&tm_d, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, g.out,
                     uint64_t(g.epi_op == HQ_EPILOGUE_SITU_QUANT ? g.n / 4
                              : (g.epi_op == HQ_EPILOGUE_IDENTITY || g.epi_op == HQ_EPILOGUE_SIGMOID) ? out_cols
                                                                                                       : out_cols / 2),
                     uint64_t(out_rows),
                     uint64_t(g.ldo) * 2, kEpiChunk, 32, CU_TENSOR_MAP_SWIZZLE_64B);
    if (!maps_ok) {
        return fail(err, errlen, HQ_ERR_CUDA, "cuTensorMapEncodeTiled failed for the GEMM operands");
    }
    int tiles_m = (g.m + kBM - 1) / kBM;
    if (g.grp.kind == kGroupBatch || g.grp.kind == kGroupMasked) {
        // (group, 128-row tile) pairs; a straddling tile counts once per group.  For the
        // masked kind this is the upper bound that sizes the grid: the kernel walks the
        // valid rows only.
        tiles_m = 0;
        for (int b = 0; b < g.grp.count; ++b) {
            tiles_m += int(((int64_t(b) + 1) * g.grp.rows - 1) / kBM - (int64_t(b) * g.grp.rows) / kBM + 1);
        }
    }
    const int tiles_n = g.n / BN;
    const int grid = min(g.sm_count, tiles_m * tiles_n);
    const int k_tiles = int(g.k_bytes / kBKBytes);
    if constexpr (BN == 64) {
        // One row of at most sm_count / 2 tiles and a long K: two CTAs per tile, half of K each.
        if (split_k_chosen(g.grp.kind, tiles_m, tiles_n, k_tiles, g.sm_count, g.epi_op)) {
            static SmemOptIn opt_in_split;
            HQ_CUDA_TRY(opt_in_split.ensure(gemm_kernel<BN, KIND, true>, C::kSmemBytes));
            HQ_CUDA_TRY(launch(gemm_kernel<BN, KIND, true>, dim3(2 * tiles_n), dim3(kThreads), size_t(C::kSmemBytes),
                               g.stream, g.pdl, 2, tm_a, tm_b, tm_d, g.sfa, g.sfb, g.alpha, g.bias, g.epi_op, g.out,
                               g.ldo, g.m, g.n, k_tiles, g.kq_dim, tiles_m, tiles_n, a_rows,
                               g.direct_store ? 1 : 0, issuers_in_order(), g.grp, g.situ));
            return HQ_OK;
        }
    }
    // One row of 64-wide dense tiles with a plain epilogue (65 to 128 activation rows, or fewer
    // when the small-M kernel is not taken): two MMA issuers with an accumulator each (see the
    // kernel).  Problems with several rows of tiles never take that mode, so that every tile
    // shape sums the k-tiles of an output element in the same order and gives the same bits.
    int dual = BN == 64 && g.grp.kind == kGroupDense && tiles_m == 1 && k_tiles >= 2 &&
                       (g.epi_op == HQ_EPILOGUE_IDENTITY || g.epi_op == HQ_EPILOGUE_SIGMOID)
                   ? 1
                   : 0;
    // Everything else: two issuers in k order (same bits as one issuer; the dense and the
    // grouped kinds alike).  HALOPS_B200_ISSUERS=1 keeps one issuer (read on every call).
    if (dual == 0 && k_tiles >= 2) dual = issuers_in_order();
    HQ_CUDA_TRY(launch(gemm_kernel<BN, KIND>, dim3(grid), dim3(kThreads), size_t(C::kSmemBytes), g.stream,
                       g.pdl, 1, tm_a, tm_b, tm_d, g.sfa, g.sfb, g.alpha, g.bias, g.epi_op, g.out, g.ldo, g.m, g.n, k_tiles,
                       g.kq_dim, tiles_m, tiles_n, a_rows, g.direct_store ? 1 : 0, dual, g.grp, g.situ));
    return HQ_OK;
}

template <int BN, int KIND, bool kGather = false, bool kGrouped = false>
int launch_pair(const GemmArgs& g, char* err, size_t errlen, __nv_bfloat16* const* gather = nullptr,
                int gather_count = 0) {
    using C = Cfg2<BN, KIND>;
    static SmemOptIn opt_in;
    int dev = 0;
    HQ_CUDA_TRY(opt_in.ensure(gemm_pair_kernel<BN, KIND, kGather, kGrouped>, C::kSmemBytes, &dev));
    // the grouped kinds: weights (and their scales) of all groups are stacked; a batch writes
    // [rows, count * N]
    const int64_t weights = kGrouped ? g.grp.count : 1;
    const int64_t out_rows = kGrouped && g.grp.kind == kGroupBatch ? g.grp.rows : g.m;
    const int64_t out_cols = kGrouped && g.grp.kind == kGroupBatch ? weights * g.n : g.n;

    const uint64_t atoms_a = uint64_t((g.m + 127) / 128) * uint64_t(g.kq_dim);
    const uint64_t atoms_b = uint64_t(weights) * uint64_t((g.n + 127) / 128) * uint64_t(g.kq_dim);
    CUtensorMap tm_a, tm_b, tm_d, tm_sfa, tm_sfb;
    const bool maps_ok =
        make_tmap_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, g.a, uint64_t(g.k_bytes), uint64_t(g.m),
                     uint64_t(g.k_bytes), kBKBytes, kBM, CU_TENSOR_MAP_SWIZZLE_128B) &&
        // (KIND 3: packed e2m1 weights, spread to one byte per value by the copy; see launch_tile)
        (KIND == 3 ? make_tmap_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, g.b, uint64_t(g.k_bytes),
                                  uint64_t(weights * g.n), uint64_t(g.k_bytes / 2), kBKBytes, BN / 2,
                                  CU_TENSOR_MAP_SWIZZLE_128B)
                   : make_tmap_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, g.b, uint64_t(g.k_bytes),
                                  uint64_t(weights * g.n), uint64_t(g.k_bytes), kBKBytes, BN / 2,
                                  CU_TENSOR_MAP_SWIZZLE_128B)) &&
        // (the gathering kernel stores boxes of two chunks, see its epilogue)
        make_tmap_2d(&tm_d, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, g.out, uint64_t(out_cols), uint64_t(out_rows),
                     uint64_t(g.ldo) * 2, kGather ? 2 * kEpiChunk : kEpiChunk, 32,
                     kGather ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B) &&
        // scale atoms as rows of 128 32-bit words
        make_tmap_2d(&tm_sfa, CU_TENSOR_MAP_DATA_TYPE_UINT32, g.sfa, 128, atoms_a, 512, 128, C::kSfKAtoms,
                     CU_TENSOR_MAP_SWIZZLE_NONE) &&
        make_tmap_2d(&tm_sfb, CU_TENSOR_MAP_DATA_TYPE_UINT32, g.sfb, 128, atoms_b, 512, 128, C::kSfKAtoms,
                     CU_TENSOR_MAP_SWIZZLE_NONE);
    if (!maps_ok) {
        return fail(err, errlen, HQ_ERR_CUDA, "cuTensorMapEncodeTiled failed for the GEMM operands");
    }
    const int tiles_m = (g.m + 255) / 256;
    const int tiles_n = g.n / BN;
    // persistent grid: no more clusters than can be resident at once
    static int max_clusters[64];
    static std::mutex max_clusters_mutex;
    std::lock_guard<std::mutex> max_clusters_lock(max_clusters_mutex);
    const int slot = dev >= 0 && dev < 64 ? dev : 63;
    if (max_clusters[slot] == 0 || dev != slot) {
        cudaLaunchConfig_t occ = {};
        occ.gridDim = dim3(2 * 74);
        occ.blockDim = dim3(C::kThreads);
        occ.dynamicSmemBytes = size_t(C::kSmemBytes);
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2;
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        occ.attrs = at;
        occ.numAttrs = 1;
        int n = 0;
        HQ_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<BN, KIND, kGather, kGrouped>, &occ));
        max_clusters[slot] = n > 0 ? n : 1;
    }
    const int clusters = min(min(g.sm_count / 2, max_clusters[slot]), tiles_m * tiles_n);
    const int k_tiles = int(g.k_bytes / kBKBytes);
    GatherMaps<kGather> peers{};
    if constexpr (kGather) {
        for (int q = 0; q < gather_count; ++q) {
            if (!make_tmap_2d(&peers.out[q], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, gather[q], uint64_t(g.n), uint64_t(g.m),
                              uint64_t(g.ldo) * 2, 2 * kEpiChunk, 32, CU_TENSOR_MAP_SWIZZLE_128B)) {
                return fail(err, errlen, HQ_ERR_CUDA, "cuTensorMapEncodeTiled failed for the output of a peer");
            }
        }
        peers.count = gather_count;
    }
    const PairGroupArgs ga{kGrouped ? g.grp : GroupParams{kGroupDense, 1, 0, nullptr}, g.out, g.ldo, g.m, g.n};
    HQ_CUDA_TRY(launch(gemm_pair_kernel<BN, KIND, kGather, kGrouped>, dim3(2 * clusters), dim3(C::kThreads),
                       size_t(C::kSmemBytes), g.stream, g.pdl, 2, tm_a, tm_b, tm_d, tm_sfa, tm_sfb, g.alpha, g.bias,
                       g.epi_op, k_tiles, g.kq_dim, tiles_m, tiles_n, peers, ga));
    return HQ_OK;
}

// Switches of the small-M kernel, for experiments and tests (HALOPS_B200_DECODE, a comma-separated
// list read on every call): "off" sends small M to the 128 x 64 tile instead, "nosplit" keeps
// every CTA on whole tiles, "split" deals every tile to several CTAs whatever the estimate says,
// "wide" also takes 65 to 128 activation rows, "nocluster" exchanges partial tiles through the
// global scratch buffer also where a cluster could do it through shared memory.
struct DecodeSwitches {
    bool off = false, nosplit = false, split = false, wide = false, nocluster = false;
};
DecodeSwitches decode_switches() {
    DecodeSwitches d;
    const char* e = getenv("HALOPS_B200_DECODE");
    if (e == nullptr) return d;
    d.off = strstr(e, "off") != nullptr;
    d.nosplit = strstr(e, "nosplit") != nullptr;
    d.split = !d.nosplit && strstr(e, "split") != nullptr;
    d.wide = strstr(e, "wide") != nullptr;
    d.nocluster = strstr(e, "nocluster") != nullptr;
    return d;
}

// Small M goes to the operand-swapped kernel: dense MXFP8 without bias, plain or sigmoid
// epilogue, no forced tile.
bool decode_eligible(int64_t m, int64_t n, int64_t k, int mode, int epi_op, bool has_bias) {
    const char* forced = getenv("HALOPS_B200_TILE");
    if (forced != nullptr && forced[0] != '\0') return false;
    if ((n / 128 + 1) * (k / 256 + 1) >= (int64_t(1) << 31)) return false;
    // Up to 64 activation rows by default.  With 65 to 128 a stage is half activations, the
    // weight in flight per CTA halves, and the 128 x 64 tile is faster (18.8 against 16.9 us on
    // 128 x 8192 x 4096); HALOPS_B200_DECODE=wide sends them here all the same.
    const DecodeSwitches sw = decode_switches();
    const int64_t m_max = sw.wide ? 128 : 64;
    return mode == HQ_MODE_W8A8_MXFP8 && m >= 1 && m <= m_max && n % 64 == 0 && k % 128 == 0 && !has_bias &&
           (epi_op == HQ_EPILOGUE_IDENTITY || epi_op == HQ_EPILOGUE_SIGMOID) && !sw.off;
}

int decode_width(int64_t m) { return m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128; }

// bytes of the operand ring of gemm_decode_kernel<NACT>: where a cluster's partial tiles land
int64_t decode_ring_bytes(int nact) {
    switch (nact) {
        case 16:
            return int64_t(DecCfg<16>::kStages) * DecCfg<16>::kWBytes;
        case 32:
            return int64_t(DecCfg<32>::kStages) * DecCfg<32>::kWBytes;
        case 64:
            return int64_t(DecCfg<64>::kStages) * DecCfg<64>::kWBytes;
        default:
            return int64_t(DecCfg<128>::kStages) * DecCfg<128>::kWBytes;
    }
}

// How many clusters of 2, 4 and 8 CTAs of gemm_decode_kernel<NACT> the current device can hold at
// once; asked once per device and width.  Without a device (shape queries on a machine without
// a GPU) the figures of a B200 stand in: 74, 36 and 14.
template <int NACT>
void decode_cluster_query(DecClusterLimits* out) {
    for (int sc = 2; sc <= 8; sc *= 2) {
        cudaLaunchConfig_t occ = {};
        occ.gridDim = dim3(unsigned(sc));
        occ.blockDim = dim3(kDecThreads);
        occ.dynamicSmemBytes = size_t(DecCfg<NACT>::kSmemBytes);
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = unsigned(sc);
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        occ.attrs = at;
        occ.numAttrs = 1;
        int n = 0;
        if (cudaFuncSetAttribute(gemm_decode_kernel<NACT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 DecCfg<NACT>::kSmemBytes) != cudaSuccess ||
            cudaOccupancyMaxActiveClusters(&n, gemm_decode_kernel<NACT>, &occ) != cudaSuccess) {
            cudaGetLastError();
            n = sc == 2 ? 74 : sc == 4 ? 36 : 14;
        }
        out->max_active[sc] = n;
    }
}

const DecClusterLimits* decode_cluster_limits(int nact) {
    static std::mutex mu;
    static DecClusterLimits limits[64][4];
    static bool known[64][4];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        dev = 63;
    }
    const int slot = dev >= 0 && dev < 64 ? dev : 63;
    const int w = nact == 16 ? 0 : nact == 32 ? 1 : nact == 64 ? 2 : 3;
    std::lock_guard<std::mutex> lock(mu);
    if (!known[slot][w]) {
        switch (nact) {
            case 16:
                decode_cluster_query<16>(&limits[slot][w]);
                break;
            case 32:
                decode_cluster_query<32>(&limits[slot][w]);
                break;
            case 64:
                decode_cluster_query<64>(&limits[slot][w]);
                break;
            default:
                decode_cluster_query<128>(&limits[slot][w]);
        }
        known[slot][w] = true;
    }
    return &limits[slot][w];
}

DecPlan decode_plan(int64_t m, int64_t n, int64_t k_bytes, int sm_count) {
    const DecodeSwitches sw = decode_switches();
    const int nact = decode_width(m);
    return dec_plan(int(n), k_bytes, sm_count, !sw.nosplit, nact, sw.split, decode_ring_bytes(nact),
                    sw.nocluster ? nullptr : decode_cluster_limits(nact));
}

template <int NACT>
int launch_decode(const GemmArgs& g, char* err, size_t errlen) {
    using C = DecCfg<NACT>;
    static SmemOptIn opt_in;
    int dev = 0;
    HQ_CUDA_TRY(opt_in.ensure(gemm_decode_kernel<NACT>, C::kSmemBytes, &dev));
    DecParams p;
    p.plan = decode_plan(g.m, g.n, g.k_bytes, g.sm_count);
    DecScratch scratch;
    if (!p.plan.aligned && p.plan.cluster <= 1 && !dec_scratch(dev, g.stream, &scratch)) {
        // no scratch buffer to be had: whole tiles per CTA need none
        p.plan.ctas = p.plan.tiles < g.sm_count ? p.plan.tiles : g.sm_count;
        p.plan.aligned = 1;
        p.plan.fits32 = 0;
    }
    const int x_rows = int((g.m + 7) / 8 * 8);
    CUtensorMap tm_w, tm_x, tm_o;
    const bool maps_ok =
        make_tmap_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, g.b, uint64_t(g.k_bytes), uint64_t(g.n),
                     uint64_t(g.k_bytes), kBKBytes, kDecRows, CU_TENSOR_MAP_SWIZZLE_128B) &&
        make_tmap_2d(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, g.a, uint64_t(g.k_bytes), uint64_t(g.m),
                     uint64_t(g.k_bytes), kBKBytes, uint32_t(x_rows), CU_TENSOR_MAP_SWIZZLE_128B) &&
        // the epilogue stores [16 rows x 32 columns] boxes; rows past M and columns past N are clipped
        make_tmap_2d(&tm_o, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, g.out, uint64_t(g.n), uint64_t(g.m),
                     uint64_t(g.ldo) * 2, 32, 16, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (!maps_ok) {
        return fail(err, errlen, HQ_ERR_CUDA, "cuTensorMapEncodeTiled failed for the GEMM operands");
    }
    p.sfw = g.sfb;
    p.early_weights = g.pdl && g.early_weights ? 1 : 0;
    p.sfx = g.sfa;
    p.scratch = scratch.partials;
    p.counters = scratch.counters;
    p.m = g.m;
    p.n = g.n;
    p.k_bytes = g.k_bytes;
    p.kq_dim = g.kq_dim;
    p.x_rows = x_rows;
    p.epi_op = g.epi_op;
    HQ_CUDA_TRY(launch(gemm_decode_kernel<NACT>, dim3(p.plan.ctas), dim3(kDecThreads), size_t(C::kSmemBytes),
                       g.stream, g.pdl, unsigned(p.plan.cluster > 1 ? p.plan.cluster : 1), tm_w, tm_x, tm_o, p));
    return HQ_OK;
}

// ---------------------------------------------------------------------------- small M without any allocation
//
// hq_dense_gemm_small_m_noalloc is for callers that cannot let a library allocate device
// memory behind their back: code that runs between the begin and end of a stream capture (a
// cudaMalloc there fails the capture), serving loops that hand all of the GPU's memory to
// their own pool at start-up and treat a later cudaMalloc as a bug, and real-time paths that
// must not take the allocator's locks.  The small-M kernel needs scratch memory when it deals
// one tile of the weight to several CTAs (float32 partial tiles and one counter per tile);
// hq_dense_gemm gets it from cudaMalloc on first use.  This variant keeps it in the array
// below, which is part of the library's image: every GPU that loads the library holds these
// bytes until the process ends, whether the entry point is called or not.
//
// Limits that keep the array modest: at most kNoAllocMaxM activation rows (32-column
// accumulators, 16 KB per partial tile), at most kNoAllocMaxCtas CTAs with two partial tiles
// each, at most kNoAllocMaxTiles weight tiles of 128 rows.
constexpr int kNoAllocMaxM = 32;
constexpr int kNoAllocMaxCtas = 160;
constexpr int kNoAllocMaxTiles = 4096;
constexpr size_t kNoAllocPartialFloats = size_t(kNoAllocMaxCtas) * 2 * 32 * kDecRows;  // 5 MiB of float32
constexpr size_t kNoAllocBytes = kNoAllocPartialFloats * sizeof(float) + size_t(kNoAllocMaxTiles) * sizeof(int);

// In host code this name is only a handle for the runtime's symbol calls; the device address
// comes from cudaGetSymbolAddress (see noalloc_scratch below).
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

// Device address of the array on the current device, looked up once per device.  The
// look-up may initialise the module on that device, so the first call on a device should
// come before any stream capture.
cudaError_t noalloc_scratch(int dev, DecScratch* out) {
    static std::mutex mu;
    static unsigned char* addr[64];
    std::lock_guard<std::mutex> lock(mu);
    unsigned char* base = dev >= 0 && dev < 64 ? addr[dev] : nullptr;
    if (base == nullptr) {
        const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&base), g_noalloc_scratch);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) addr[dev] = base;
    }
    out->partials = reinterpret_cast<float*>(base);
    out->counters = reinterpret_cast<int*>(base + kNoAllocPartialFloats * sizeof(float));
    return cudaSuccess;
}

template <int NACT>
int launch_decode_noalloc(const GemmArgs& g, const DecPlan& plan, char* err, size_t errlen) {
    using C = DecCfg<NACT>;
    static SmemOptIn opt_in;
    int dev = 0;
    HQ_CUDA_TRY(opt_in.ensure(gemm_decode_kernel<NACT>, C::kSmemBytes, &dev));
    DecScratch scratch;
    HQ_CUDA_TRY(noalloc_scratch(dev, &scratch));
    DecParams p;
    p.plan = plan;
    if (!plan.aligned) {
        // The array keeps what the last call left in it.  The partial tiles are written before
        // they are read; the tile counters must start at zero, and a call that was cut short
        // may have left some counted: clear the ones this launch uses, in stream order.
        HQ_CUDA_TRY(cudaMemsetAsync(scratch.counters, 0, size_t(plan.tiles) * sizeof(int), g.stream));
    }
    const int x_rows = int((g.m + 7) / 8 * 8);
    CUtensorMap tm_w, tm_x, tm_o;
    const bool maps_ok =
        make_tmap_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, g.b, uint64_t(g.k_bytes), uint64_t(g.n),
                     uint64_t(g.k_bytes), kBKBytes, kDecRows, CU_TENSOR_MAP_SWIZZLE_128B) &&
        make_tmap_2d(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, g.a, uint64_t(g.k_bytes), uint64_t(g.m),
                     uint64_t(g.k_bytes), kBKBytes, uint32_t(x_rows), CU_TENSOR_MAP_SWIZZLE_128B) &&
        make_tmap_2d(&tm_o, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, g.out, uint64_t(g.n), uint64_t(g.m),
                     uint64_t(g.ldo) * 2, 32, 16, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (!maps_ok) {
        return fail(err, errlen, HQ_ERR_CUDA, "cuTensorMapEncodeTiled failed for the GEMM operands");
    }
    p.sfw = g.sfb;
    p.early_weights = g.pdl && g.early_weights ? 1 : 0;
    p.sfx = g.sfa;
    p.scratch = scratch.partials;
    p.counters = scratch.counters;
    p.m = g.m;
    p.n = g.n;
    p.k_bytes = g.k_bytes;
    p.kq_dim = g.kq_dim;
    p.x_rows = x_rows;
    p.epi_op = g.epi_op;
    HQ_CUDA_TRY(launch(gemm_decode_kernel<NACT>, dim3(plan.ctas), dim3(kDecThreads), size_t(C::kSmemBytes), g.stream,
                       g.pdl, unsigned(plan.cluster > 1 ? plan.cluster : 1), tm_w, tm_x, tm_o, p));
    return HQ_OK;
}

const char* mode_name(int mode) {
    switch (mode) {
        case HQ_MODE_W8A8_MXFP8:
            return "w8a8-mxfp8";
        case HQ_MODE_W4A4_MXFP4:
            return "w4a4-mxfp4";
        case HQ_MODE_W4A8_MXFP4:
            return "w4a8-mxfp4";
        default:
            return "w4a4-nvfp4";
    }
}

struct TilePick {
    int bn;     // tile width, 0 = no tile fits
    bool pair;  // 256-row tile on a pair of CTAs
};

// Shape legality follows the reference's "some compiled tile fits" rule
// (csrc/kernel/gemm/gemm_dispatch.cuh:65-100 over the tiles of gemm_tile.cuh:371-395):
// MXFP8 needs K % 128 == 0 and N % 64 == 0, the FP4 modes K % 256 == 0 and
// N % 128 == 0; any M >= 1.  Among the legal tiles: the largest that still
// gives every SM (or SM pair) a tile; failing that, the narrowest single-CTA
// tile that divides N (most CTAs streaming the weight).  HALOPS_B200_TILE
// (pair256 | pair128 | 256 | 128 | 64) overrides the choice when it is legal.
TilePick pick_tile(int64_t m, int64_t n, int64_t k, int mode, int sm_count) {
    // (FP8 activations x FP4 weights tile like FP8: 128 values of K per k-tile)
    const bool fp8 = mode == HQ_MODE_W8A8_MXFP8 || mode == HQ_MODE_W4A8_MXFP4;
    if (m < 1 || n < 1 || k < 1) return {0, false};
    if (fp8 ? (k % 128 != 0 || n % 64 != 0) : (k % 256 != 0 || n % 128 != 0)) return {0, false};
    const int64_t tiles_m = (m + kBM - 1) / kBM;
    const int64_t tiles_m2 = (m + 255) / 256;
    const char* forced = getenv("HALOPS_B200_TILE");
    if (forced != nullptr && forced[0] != '\0') {
        const bool pair = strncmp(forced, "pair", 4) == 0;
        const int w = atoi(pair ? forced + 4 : forced);
        const bool legal = (w == 256 || w == 128 || (w == 64 && fp8 && !pair)) && n % w == 0;
        if (legal) return {w, pair};
    }
    if (tiles_m == 1) {
        // One row of tiles: the weight streams through once, so what counts is the
        // largest share of weight rows any CTA has to stream (tiles per CTA x width,
        // plus a fixed cost per tile of about 16 rows' worth); ties go to the wider tile.
        int best = 0;
        int64_t best_cost = 0;
        for (int w : {256, 128, 64}) {
            if (n % w != 0 || (w == 64 && !fp8)) continue;
            const int64_t tiles = n / w;
            const int64_t cost = ((tiles + sm_count - 1) / sm_count) * (w + 16);
            if (best == 0 || cost < best_cost) {
                best = w;
                best_cost = cost;
            }
        }
        return {best, false};
    }
    // Several rows of tiles: waves x time per tile.  Fitted to this build's kernels on B200
    // (MXFP8; M = N = K = 8192, 8192 x 4096 x 4096 and 4096 x 14336 x 4096): a tile costs its
    // k-tiles plus a fixed number of k-tile times for fill, drain and the hand-over to the
    // next tile.  128x256: 0.46 us per k-tile + 2 (425 / 109.5 / 199 us); 256x256 pair:
    // 0.404 + 3.2 (380 / 99.5 / 173 us); 128x128 0.35 (650 us); 256x128 pair 0.348 (633 us);
    // 128x64 is extrapolated.  (These fits were made with one MMA issuer in the single-CTA kernel;
    // its second, in-order issuer shortens the narrow and the FP4 tiles more than the choices made
    // here depend on.)  The FP4 kinds stay on single-CTA tiles: the pair measured no
    // faster there (126 against 113 us on 4096 x 14336 x 4096 with the same scale path).
    struct Cand {
        int bn;
        bool pair;
        double us_per_ktile;
        double extra_ktiles;
    };
    const Cand cands[5] = {{256, false, 0.46, 2.0}, {256, true, 0.404, 3.2}, {128, false, 0.35, 1.0},
                           {128, true, 0.348, 1.0},  {64, false, 0.27, 1.0}};
    const double k_tiles = double(k) / (fp8 ? 128.0 : 256.0);
    TilePick best = {0, false};
    double best_cost = 0.0;
    for (const Cand& c : cands) {
        if (n % c.bn != 0 || (c.bn == 64 && !fp8) || (c.pair && (m <= kBM || !fp8))) continue;
        const int64_t tiles = (c.pair ? tiles_m2 : tiles_m) * (n / c.bn);
        const int64_t units = c.pair ? sm_count / 2 : sm_count;
        if (units < 1) continue;
        const double waves = double((tiles + units - 1) / units);
        const double cost = waves * (k_tiles + c.extra_ktiles) * c.us_per_ktile;
        if (best.bn == 0 || cost < best_cost * 0.999) {
            best = {c.bn, c.pair};
            best_cost = cost;
        }
    }
    return best;
}

std::mutex g_sm_mutex;
int g_sm_cache[64];

}  // namespace
}  // namespace hq

extern "C" int hq_sm_count(int device) {
    if (device < 0 || device >= 64) {
        if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
    }
    std::lock_guard<std::mutex> lock(hq::g_sm_mutex);
    if (hq::g_sm_cache[device] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
        hq::g_sm_cache[device] = n;
    }
    return hq::g_sm_cache[device];
}

extern "C" int hq_describe_tile(int64_t m, int64_t n, int64_t k, int mode, int sm_count, int device,
                                char* buf, size_t buflen) {
    if (hq_group_size(mode) == 0) return hq::fail(buf, buflen, HQ_ERR_INVALID, "Unsupported mode: %d", mode);
    const int sm = sm_count > 0 ? sm_count : hq_sm_count(device);
    const hq::TilePick pick = hq::pick_tile(m, n, k, mode, sm > 0 ? sm : 148);
    if (pick.bn == 0) {
        return hq::fail(buf, buflen, HQ_ERR_INVALID,
                        "No dense %s tile for M=%lld (grid M=%lld), N=%lld, K=%lld", hq::mode_name(mode),
                        (long long)(m < 128 ? m : hq_sf_rows(m)), (long long)(m < 128 ? m : hq_sf_rows(m)), (long long)n,
                        (long long)k);
    }
    if (hq::decode_eligible(m, n, k, mode, HQ_EPILOGUE_IDENTITY, false)) {
        const hq::DecPlan plan = hq::decode_plan(m, n, k, sm > 0 ? sm : 148);
        if (buf != nullptr && buflen > 0) {
            snprintf(buf, buflen,
                     "[gemm] mode=dense kind=%s m=%lld n=%lld k=%lld sm=%d -> swap 128x%d/256 pair=0 splitk=%d ctas=%d cluster=%d",
                     hq::mode_name(mode), (long long)m, (long long)n, (long long)k, sm, hq::decode_width(m),
                     plan.aligned ? 0 : 1, plan.ctas, plan.cluster > 1 ? plan.cluster : 1);
        }
        return HQ_OK;
    }
    if (buf != nullptr && buflen > 0) {
        // (the Identity epilogue is assumed for the split-K note)
        const bool split = pick.bn == 64 && !pick.pair &&
                           hq::split_k_chosen(hq::kGroupDense, int((m + hq::kBM - 1) / hq::kBM), int(n / 64),
                                              int(k / 128), sm > 0 ? sm : 148, HQ_EPILOGUE_IDENTITY);
        snprintf(buf, buflen, "[gemm] mode=dense kind=%s m=%lld n=%lld k=%lld sm=%d -> %dx%d/%d pair=%d splitk=%d",
                 hq::mode_name(mode), (long long)m, (long long)n, (long long)k, sm, pick.pair ? 256 : hq::kBM,
                 pick.bn, mode == HQ_MODE_W8A8_MXFP8 ? 128 : 256, pick.pair ? 1 : 0, split ? 1 : 0);
    }
    return HQ_OK;
}

namespace hq {
namespace {

// Shared body of the GEMM entry points.  `situ` is null except for the SiTU-GLU
// quantising epilogue, whose outputs it names (then `out` / `ldo` are unused).
int dense_gemm_impl(const void* a, const void* b, const void* sfa, const void* sfb, void* out, const void* bias,
                    const float* alpha, int64_t m, int64_t n, int64_t k, int64_t sfa_bytes, int64_t sfb_bytes,
                    int64_t ldo, int mode, int epilogue, const SituParams* situ, int sm_count, int use_pdl,
                    int device, void* stream, char* err, size_t errlen) {
    const int group = hq_group_size(mode);
    if (group == 0) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "Unsupported mode: %d. Expected 'w8a8-mxfp8', 'w4a4-mxfp4' or 'w4a4-nvfp4'.", mode);
    }
    const bool is_situ = epilogue == HQ_EPILOGUE_SITU_QUANT && situ != nullptr;
    if (epilogue != HQ_EPILOGUE_IDENTITY && epilogue != HQ_EPILOGUE_SIGMOID && !is_situ) {
        return fail(err, errlen, HQ_ERR_UNSUPPORTED, "Unsupported epilogue %d for %s", epilogue,
                    hq::mode_name(mode));
    }
    if (is_situ && mode != HQ_MODE_W8A8_MXFP8) {
        return fail(err, errlen, HQ_ERR_UNSUPPORTED, "Unsupported epilogue %d for %s", epilogue,
                    hq::mode_name(mode));
    }
    if (bias != nullptr && mode != HQ_MODE_W8A8_MXFP8) {
        return fail(err, errlen, HQ_ERR_INVALID, "W4A4 mode does not support bias yet.");
    }
    if (bias != nullptr && !is_situ && m % 256 != 0) {
        // kept from the reference, whose bias tile has no per-row store predicate
        return fail(err, errlen, HQ_ERR_INVALID,
                    "the bias tile has no per-row store predicate yet, so M must be a multiple of 256 "
                    "when bias is given, got %lld", (long long)m);
    }
    if (bias != nullptr && !hq::aligned(bias, 16)) {
        return fail(err, errlen, HQ_ERR_INVALID, "bias must be 16-byte aligned");
    }
    if (m < 0 || n < 0 || k < 0 || m > INT32_MAX || n > INT32_MAX || k > INT32_MAX) {
        return fail(err, errlen, HQ_ERR_INVALID, "input must be a 2D tensor of shape [M, K]");
    }
    if (mode == HQ_MODE_W4A4_MXFP4 && alpha != nullptr) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "'w4a4-mxfp4' does not take alpha; the global scaling factor is only used by "
                    "'w4a4-nvfp4'.");
    }
    if (mode == HQ_MODE_W4A4_NVFP4 && alpha == nullptr) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "W4A4-nvfp4 mode requires alpha input (per-batch scaling).");
    }
    if (m == 0 || n == 0) return HQ_OK;

    // shape legality first: it needs no device
    if (hq::pick_tile(m, n, k, mode, 148).bn == 0) {
        return fail(err, errlen, HQ_ERR_INVALID, "No dense %s tile for M=%lld (grid M=%lld), N=%lld, K=%lld",
                    hq::mode_name(mode), (long long)(m < 128 ? m : hq_sf_rows(m)),
                    (long long)(m < 128 ? m : hq_sf_rows(m)), (long long)n, (long long)k);
    }
    const int64_t sf_k = k / group;
    const int64_t need_a = hq_sf_rows(m) * sf_k;
    const int64_t need_b = hq_sf_rows(n) * sf_k;
    if (sfa_bytes < need_a) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "sfa must hold whole 128-row SfAtoms: expected at least %lld elements (%lld x %lld) "
                    "for M=%lld, got %lld",
                    (long long)need_a, (long long)hq_sf_rows(m), (long long)sf_k, (long long)m,
                    (long long)sfa_bytes);
    }
    if (sfb_bytes < need_b) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "sfb must hold whole 128-row SfAtoms: expected at least %lld elements (%lld x %lld) "
                    "for N=%lld, got %lld",
                    (long long)need_b, (long long)hq_sf_rows(n), (long long)sf_k, (long long)n,
                    (long long)sfb_bytes);
    }
    const hq::DeviceGuard guard(device);
    if (!guard.ok()) return fail(err, errlen, HQ_ERR_CUDA, "cannot select CUDA device %d", device);
    const int sm_all = hq_sm_count(device);
    const int sm = sm_count > 0 ? (sm_count < sm_all || sm_all == 0 ? sm_count : sm_all) : sm_all;
    if (sm <= 0) return fail(err, errlen, HQ_ERR_CUDA, "cannot query the SM count of device %d", device);
    hq::TilePick pick = hq::pick_tile(m, n, k, mode, sm);
    if (is_situ) {
        // the quantising epilogue lives in the single-CTA kernel
        pick.pair = false;
        out = situ->q;
        ldo = situ->ldq / 2;
    }
    if (a == nullptr || b == nullptr || sfa == nullptr || sfb == nullptr || out == nullptr) {
        return fail(err, errlen, HQ_ERR_INVALID, "null pointer argument");
    }
    if (!hq::aligned(a, 16) || !hq::aligned(b, 16) || !hq::aligned(sfa, 16) || !hq::aligned(sfb, 16) ||
        !hq::aligned(out, 16) || ldo < (is_situ ? n / 4 : n) || ldo % 8 != 0) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "operands, scales and output must be 16-byte aligned and the output row stride a "
                    "multiple of 8 elements");
    }

    hq::GemmArgs g;
    g.a = a;
    g.b = b;
    g.sfa = static_cast<const uint8_t*>(sfa);
    g.sfb = static_cast<const uint8_t*>(sfb);
    g.alpha = alpha;
    g.bias = static_cast<const __nv_bfloat16*>(bias);
    g.epi_op = epilogue;
    g.situ = is_situ ? *situ : hq::SituParams{};
    g.out = static_cast<__nv_bfloat16*>(out);
    g.ldo = ldo;
    g.m = int(m);
    g.n = int(n);
    g.grp = hq::GroupParams{hq::kGroupDense, 1, 0, nullptr};
    g.k_bytes = mode == HQ_MODE_W8A8_MXFP8 ? k : k / 2;
    g.kq_dim = int(sf_k / 4);
    g.sm_count = sm;
    g.pdl = use_pdl != 0;
    g.early_weights = use_pdl == 2;
    {
        // test switch, read on every call: store every tile from registers
        const char* e = getenv("HALOPS_B200_EPILOGUE");
        g.direct_store = e != nullptr && strcmp(e, "direct") == 0;
    }
    g.stream = static_cast<cudaStream_t>(stream);

    if (!is_situ && hq::decode_eligible(m, n, k, mode, epilogue, bias != nullptr)) {
        switch (hq::decode_width(m)) {
            case 16:
                return hq::launch_decode<16>(g, err, errlen);
            case 32:
                return hq::launch_decode<32>(g, err, errlen);
            case 64:
                return hq::launch_decode<64>(g, err, errlen);
            default:
                return hq::launch_decode<128>(g, err, errlen);
        }
    }

#define HQ_DISPATCH(KIND)                                                            \
    if (pick.pair) {                                                                 \
        return pick.bn == 256 ? hq::launch_pair<256, KIND>(g, err, errlen)           \
                              : hq::launch_pair<128, KIND>(g, err, errlen);          \
    }                                                                                \
    switch (pick.bn) {                                                               \
        case 256:                                                                    \
            return hq::launch_tile<256, KIND>(g, err, errlen);                       \
        case 128:                                                                    \
            return hq::launch_tile<128, KIND>(g, err, errlen);                       \
        default:                                                                     \
            return hq::launch_tile<64, KIND>(g, err, errlen);                        \
    }
    if (mode == HQ_MODE_W8A8_MXFP8) {
        HQ_DISPATCH(0)
    } else if (mode == HQ_MODE_W4A4_NVFP4) {
        HQ_DISPATCH(1)
    } else {
        HQ_DISPATCH(2)
    }
#undef HQ_DISPATCH
}

}  // namespace
}  // namespace hq

extern "C" int hq_dense_gemm(const void* a, const void* b, const void* sfa, const void* sfb, void* out,
                             const void* bias, const float* alpha, int64_t m, int64_t n, int64_t k, int64_t sfa_bytes,
                             int64_t sfb_bytes, int64_t ldo, int mode, int epilogue, int sm_count,
                             int use_pdl, int device, void* stream, char* err, size_t errlen) {
    return hq::dense_gemm_impl(a, b, sfa, sfb, out, bias, alpha, m, n, k, sfa_bytes, sfb_bytes, ldo, mode,
                               epilogue, nullptr, sm_count, use_pdl, device, stream, err, errlen);
}

extern "C" int hq_dense_gemm_situ_quant(const void* a, const void* b, const void* sfa, const void* sfb,
                                        void* out_q, void* out_sf, const void* bias, int64_t m, int64_t n,
                                        int64_t k, int64_t sfa_bytes, int64_t sfb_bytes, int64_t out_sf_bytes,
                                        float situ_beta, float situ_linear_beta, int sm_count, int use_pdl,
                                        int device, void* stream, char* err, size_t errlen) {
    // N / 2 / 32 output scale columns must fill whole SfAtoms (4 columns)
    if (n % 256 != 0) {
        return hq::fail(err, errlen, HQ_ERR_INVALID,
                        "No dense w8a8-mxfp8 tile for M=%lld (grid M=%lld), N=%lld, K=%lld", (long long)m,
                        (long long)m, (long long)n, (long long)k);
    }
    if (!(situ_beta > 0.0f) || situ_linear_beta < 0.0f) {
        return hq::fail(err, errlen, HQ_ERR_INVALID, "situ_beta must be positive and situ_linear_beta non-negative");
    }
    const int64_t kb_out = n / 2 / 32;
    if (out_q == nullptr || out_sf == nullptr || out_sf_bytes < hq_sf_rows(m) * kb_out) {
        return hq::fail(err, errlen, HQ_ERR_INVALID,
                        "output_sf must hold whole 128-row SfAtoms: expected at least %lld bytes, got %lld",
                        (long long)(hq_sf_rows(m) * kb_out), (long long)out_sf_bytes);
    }
    hq::SituParams sp{};
    sp.q = static_cast<uint8_t*>(out_q);
    sp.sf = static_cast<uint8_t*>(out_sf);
    sp.ldq = n / 2;
    sp.kb_out = int(kb_out);
    sp.beta = situ_beta;
    sp.inv_beta = 1.0f / situ_beta;
    sp.lin = situ_linear_beta;
    sp.inv_lin = situ_linear_beta != 0.0f ? 1.0f / situ_linear_beta : 0.0f;
    sp.valid_rows = int(m);
    return hq::dense_gemm_impl(a, b, sfa, sfb, out_q, bias, nullptr, m, n, k, sfa_bytes, sfb_bytes, n / 4,
                               HQ_MODE_W8A8_MXFP8, HQ_EPILOGUE_SITU_QUANT, &sp, sm_count, use_pdl, device, stream,
                               err, errlen);
}

namespace hq {
namespace {

const char* group_kind_name(int kind) {
    return kind == kGroupBatch ? "batch" : kind == kGroupMasked ? "masked" : "contiguous";
}

// The grouped kinds run in the single-CTA kernel.  `rows` = rows per group (batch,
// masked) or the mean rows per expert (contiguous), `total_m` = all rows of A.  The
// waves are sized by the (group, row tile) pairs, which exceed the row tiles of the
// stacked rows when tiles straddle groups.  Batches take any row count (straddling
// tiles are worked once per batch); the expert kinds want slots / runs that are
// multiples of 64 rows, the finest granularity of the reference's tiles
// (csrc/kernel/gemm/gemm_dispatch.cuh:65-100).
TilePick pick_tile_grouped(int kind, int64_t count, int64_t rows, int64_t total_m, int64_t n, int64_t k, int mode,
                           int sm_count, bool plain_epilogue = true) {
    if (count < 1 || rows < 1) return {0, false};
    if (kind == kGroupMasked && rows % 64 != 0) return {0, false};
    if (kind == kGroupContiguous && total_m % 64 != 0) return {0, false};
    const int64_t pad = kind != kGroupContiguous && rows % kBM != 0 ? (count - 1) * kBM : 0;
    TilePick pick = pick_tile(total_m + pad, n, k, mode, sm_count);
    // The 2-CTA tile: MXFP8 (or e4m3 x MXFP4) with a plain epilogue, and no 256-row tile may hold rows of two
    // batches or expert slots (the contiguous layout is worked per run of experts, see
    // PairWorkIter).  Otherwise a forced or modelled pair choice falls back to the same width.
    const bool whole_tiles = kind == kGroupContiguous ? total_m % 256 == 0 : rows % 256 == 0;
    const bool fp8_kind = mode == HQ_MODE_W8A8_MXFP8 || (mode == HQ_MODE_W4A8_MXFP4 && kind != kGroupBatch);
    if (!(fp8_kind && plain_epilogue && whole_tiles)) pick.pair = false;
    return pick;
}

int no_group_tile(char* err, size_t errlen, int kind, int mode, int64_t rows, int64_t total_m, int64_t n,
                  int64_t k) {
    return fail(err, errlen, HQ_ERR_INVALID, "No %s %s tile for M=%lld (grid M=%lld), N=%lld, K=%lld",
                group_kind_name(kind), mode_name(mode), (long long)rows, (long long)total_m, (long long)n,
                (long long)k);
}

// Shared body of the batch / masked / contiguous entry points.
int grouped_gemm_impl(int kind, const void* a, const void* b, const void* sfa, const void* sfb, void* out,
                      const void* bias, const float* alpha, const int* table, int64_t count, int64_t rows,
                      int64_t total_m, int64_t n, int64_t k, int64_t sfa_bytes, int64_t sfb_bytes, int64_t ldo,
                      int mode, int epilogue, const SituParams* quant, int sm_count, int use_pdl, int device,
                      void* stream, char* err, size_t errlen) {
    const bool batch = kind == kGroupBatch;
    const char* const per = batch ? "per-batch" : "per-expert";
    // FP8 activations x MXFP4 weights (UE8M0 scales per 32 on both): the expert kinds only
    const bool w4a8 = mode == HQ_MODE_W4A8_MXFP4 && !batch;
    const int group = w4a8 ? 32 : hq_group_size(mode);
    if (group == 0) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "Unsupported mode: %d. Expected 'w8a8-mxfp8', 'w4a4-nvfp4', 'w4a4-mxfp4' or 'w4a8-mxfp4'.", mode);
    }
    if (w4a8 && bias != nullptr) return fail(err, errlen, HQ_ERR_INVALID, "W4A8 mode does not support bias yet.");
    if (w4a8 && alpha != nullptr) {
        return fail(err, errlen, HQ_ERR_INVALID, "W4A8 mode does not take alpha; scales are per-group UE8M0.");
    }
    if (count < 0 || rows < 0 || total_m < 0 || n < 0 || k < 0 || total_m > INT32_MAX || count * n > INT32_MAX ||
        k > INT32_MAX) {
        return fail(err, errlen, HQ_ERR_INVALID, "problem sizes must be non-negative and below 2^31");
    }
    const bool quant_epi = epilogue == HQ_EPILOGUE_QUANT || epilogue == HQ_EPILOGUE_GATE_MUL_QUANT ||
                           epilogue == HQ_EPILOGUE_SIGMOID_GATE_MUL_QUANT;
    if (epilogue != HQ_EPILOGUE_IDENTITY && !(quant_epi && quant != nullptr && batch && mode == HQ_MODE_W8A8_MXFP8)) {
        return fail(err, errlen, HQ_ERR_UNSUPPORTED, "Unsupported epilogue %d for %s", epilogue, mode_name(mode));
    }
    if (quant_epi) {
        out = quant->q;
        ldo = quant->ldq / 2;
    }
    if (bias != nullptr && mode != HQ_MODE_W8A8_MXFP8) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    batch ? "W4A4 batch GEMM does not support bias yet." : "W4A4 mode does not support bias yet.");
    }
    if (bias != nullptr && !aligned(bias, 16)) {
        return fail(err, errlen, HQ_ERR_INVALID, "bias must be 16-byte aligned");
    }
    if (mode == HQ_MODE_W4A4_MXFP4 && alpha != nullptr) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "'w4a4-mxfp4' does not take alpha; the %s scaling factor is only used by 'w4a4-nvfp4'.", per);
    }
    if (mode == HQ_MODE_W4A4_NVFP4 && alpha == nullptr) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    batch ? "W4A4-nvfp4 mode requires alpha input (per-batch scaling)."
                          : "W4A4-nvfp4 mode requires alpha input (per-expert scaling factor).");
    }
    if (count == 0 || total_m == 0 || n == 0) return HQ_OK;
    if (pick_tile_grouped(kind, count, rows, total_m, n, k, mode, 148).bn == 0) {
        return no_group_tile(err, errlen, kind, mode, rows, total_m, n, k);
    }
    const int64_t sf_k = k / group;
    const int64_t need_a = hq_sf_rows(total_m) * sf_k;
    const int64_t need_b = count * hq_sf_rows(n) * sf_k;
    if (sfa_bytes < need_a) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "sfa must hold whole 128-row SfAtoms over the stacked rows: expected at least %lld "
                    "elements (%lld x %lld) for M=%lld, got %lld",
                    (long long)need_a, (long long)hq_sf_rows(total_m), (long long)sf_k, (long long)total_m,
                    (long long)sfa_bytes);
    }
    if (sfb_bytes < need_b) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "sfb must hold whole 128-row SfAtoms per weight: expected at least %lld elements "
                    "(%lld x %lld x %lld) for N=%lld, got %lld",
                    (long long)need_b, (long long)count, (long long)hq_sf_rows(n), (long long)sf_k, (long long)n,
                    (long long)sfb_bytes);
    }
    const DeviceGuard guard(device);
    if (!guard.ok()) return fail(err, errlen, HQ_ERR_CUDA, "cannot select CUDA device %d", device);
    const int sm_all = hq_sm_count(device);
    const int sm = sm_count > 0 ? (sm_count < sm_all || sm_all == 0 ? sm_count : sm_all) : sm_all;
    if (sm <= 0) return fail(err, errlen, HQ_ERR_CUDA, "cannot query the SM count of device %d", device);
    if (a == nullptr || b == nullptr || sfa == nullptr || sfb == nullptr || out == nullptr ||
        (!batch && table == nullptr)) {
        return fail(err, errlen, HQ_ERR_INVALID, "null pointer argument");
    }
    const int64_t out_cols = batch ? count * n : n;
    if (!aligned(a, 16) || !aligned(b, 16) || !aligned(sfa, 16) || !aligned(sfb, 16) || !aligned(out, 16) ||
        !aligned(table, 4) || ldo < (quant_epi ? out_cols / 2 : out_cols) || ldo % 8 != 0) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "operands, scales and output must be 16-byte aligned and the output row stride a "
                    "multiple of 8 elements");
    }
    const TilePick pick = pick_tile_grouped(kind, count, rows, total_m, n, k, mode, sm,
                                            epilogue == HQ_EPILOGUE_IDENTITY && !quant_epi);

    GemmArgs g;
    g.a = a;
    g.b = b;
    g.sfa = static_cast<const uint8_t*>(sfa);
    g.sfb = static_cast<const uint8_t*>(sfb);
    g.alpha = alpha;
    g.bias = static_cast<const __nv_bfloat16*>(bias);
    g.epi_op = epilogue;
    g.situ = quant_epi ? *quant : SituParams{};
    g.out = static_cast<__nv_bfloat16*>(out);
    g.ldo = ldo;
    g.m = int(total_m);
    g.n = int(n);
    g.grp = GroupParams{kind, int(count), int(rows), table};
    g.k_bytes = (mode == HQ_MODE_W8A8_MXFP8 || w4a8) ? k : k / 2;  // bytes of one A row
    g.kq_dim = int(sf_k / 4);
    g.sm_count = sm;
    g.pdl = use_pdl != 0;
    g.direct_store = false;
    g.stream = static_cast<cudaStream_t>(stream);
#define HQ_DISPATCH(KIND)                                      \
    switch (pick.bn) {                                         \
        case 256:                                              \
            return launch_tile<256, KIND>(g, err, errlen);     \
        case 128:                                              \
            return launch_tile<128, KIND>(g, err, errlen);     \
        default:                                               \
            return launch_tile<64, KIND>(g, err, errlen);      \
    }
    if (pick.pair && w4a8) {
        return pick.bn == 256 ? launch_pair<256, 3, false, true>(g, err, errlen)
                              : launch_pair<128, 3, false, true>(g, err, errlen);
    }
    if (pick.pair) {
        return pick.bn == 256 ? launch_pair<256, 0, false, true>(g, err, errlen)
                              : launch_pair<128, 0, false, true>(g, err, errlen);
    }
    if (mode == HQ_MODE_W8A8_MXFP8) {
        HQ_DISPATCH(0)
    } else if (w4a8) {
        HQ_DISPATCH(3)
    } else if (mode == HQ_MODE_W4A4_NVFP4) {
        HQ_DISPATCH(1)
    } else {
        HQ_DISPATCH(2)
    }
#undef HQ_DISPATCH
}

}  // namespace
}  // namespace hq

extern "C" int hq_describe_group_tile(int kind, int64_t count, int64_t rows, int64_t total_m, int64_t n, int64_t k,
                                      int mode, int sm_count, int device, char* buf, size_t buflen) {
    if (hq_group_size(mode) == 0 && !(mode == HQ_MODE_W4A8_MXFP4 && kind != hq::kGroupBatch)) {
        return hq::fail(buf, buflen, HQ_ERR_INVALID, "Unsupported mode: %d", mode);
    }
    if (kind < hq::kGroupBatch || kind > hq::kGroupContiguous) {
        return hq::fail(buf, buflen, HQ_ERR_INVALID, "Unsupported group kind: %d", kind);
    }
    const int sm = sm_count > 0 ? sm_count : hq_sm_count(device);
    const hq::TilePick pick = hq::pick_tile_grouped(kind, count, rows, total_m, n, k, mode, sm > 0 ? sm : 148);
    if (pick.bn == 0) return hq::no_group_tile(buf, buflen, kind, mode, rows, total_m, n, k);
    if (buf != nullptr && buflen > 0) {
        // (the Identity epilogue is assumed)
        snprintf(buf, buflen, "[gemm] mode=%s kind=%s groups=%lld m=%lld grid_m=%lld n=%lld k=%lld sm=%d -> %dx%d/%d pair=%d",
                 hq::group_kind_name(kind), hq::mode_name(mode), (long long)count, (long long)rows,
                 (long long)total_m, (long long)n, (long long)k, sm, pick.pair ? 256 : hq::kBM, pick.bn,
                 mode == HQ_MODE_W8A8_MXFP8 ? 128 : 256, pick.pair ? 1 : 0);
    }
    return HQ_OK;
}

extern "C" int hq_batch_gemm(const void* a, const void* b, const void* sfa, const void* sfb, void* out,
                             const void* bias, const float* alpha, int64_t batches, int64_t m, int64_t n,
                             int64_t k, int64_t sfa_bytes, int64_t sfb_bytes, int64_t ldo, int mode, int epilogue,
                             int sm_count, int use_pdl, int device, void* stream, char* err, size_t errlen) {
    return hq::grouped_gemm_impl(hq::kGroupBatch, a, b, sfa, sfb, out, bias, alpha, nullptr, batches, m,
                                 batches * m, n, k, sfa_bytes, sfb_bytes, ldo, mode, epilogue, nullptr, sm_count, use_pdl,
                                 device, stream, err, errlen);
}

extern "C" int hq_batch_gemm_quant(const void* a, const void* b, const void* sfa, const void* sfb, void* out_q,
                                   void* out_sf, const void* gate, int64_t gate_ld, const void* bias,
                                   int64_t batches, int64_t m, int64_t n, int64_t k, int64_t sfa_bytes,
                                   int64_t sfb_bytes, int64_t ldq, int64_t out_sf_bytes, int epilogue, int sm_count,
                                   int use_pdl, int device, void* stream, char* err, size_t errlen) {
    using hq::fail;
    const bool gated = epilogue == HQ_EPILOGUE_GATE_MUL_QUANT || epilogue == HQ_EPILOGUE_SIGMOID_GATE_MUL_QUANT;
    if (epilogue != HQ_EPILOGUE_QUANT && !gated) {
        return fail(err, errlen, HQ_ERR_INVALID, "Unsupported epilogue %d for w8a8-mxfp8", epilogue);
    }
    if (n % 128 != 0) {
        return fail(err, errlen, HQ_ERR_INVALID, "quantized output needs N %% 128 == 0, got %lld", (long long)n);
    }
    if (gated && gate == nullptr) return fail(err, errlen, HQ_ERR_INVALID, "GateMulQuant epilogues need gate");
    if (batches < 0 || m < 0 || n < 0 || batches * n > INT32_MAX) {
        return fail(err, errlen, HQ_ERR_INVALID, "input must be a 3D tensor of shape [B, M, K]");
    }
    const int64_t kb_out = batches * n / 32;
    if (batches > 0 && m > 0 && n > 0) {
        if (out_q == nullptr || out_sf == nullptr || out_sf_bytes < hq_sf_rows(m) * kb_out) {
            return fail(err, errlen, HQ_ERR_INVALID,
                        "output_sf must hold whole 128-row SfAtoms: expected at least %lld bytes, got %lld",
                        (long long)(hq_sf_rows(m) * kb_out), (long long)out_sf_bytes);
        }
        if (ldq % 16 != 0 || ldq < batches * n || !hq::aligned(out_q, 16)) {
            return fail(err, errlen, HQ_ERR_INVALID,
                        "the quantized output must be 16-byte aligned with a row stride that is a multiple of 16");
        }
        if (gated && (!hq::aligned(gate, 32) || gate_ld * 2 % 32 != 0 || gate_ld < batches * n)) {
            return fail(err, errlen, HQ_ERR_INVALID, "gate rows must be contiguous and 32-byte aligned");
        }
    }
    hq::SituParams sp{};
    sp.q = static_cast<uint8_t*>(out_q);
    sp.sf = static_cast<uint8_t*>(out_sf);
    sp.ldq = ldq;
    sp.kb_out = int(kb_out);
    sp.gate = static_cast<const __nv_bfloat16*>(gate);
    sp.gate_ld = gate_ld;
    sp.valid_rows = int(m);
    return hq::grouped_gemm_impl(hq::kGroupBatch, a, b, sfa, sfb, out_q, bias, nullptr, nullptr, batches, m,
                                 batches * m, n, k, sfa_bytes, sfb_bytes, ldq / 2, HQ_MODE_W8A8_MXFP8, epilogue, &sp,
                                 sm_count, use_pdl, device, stream, err, errlen);
}

extern "C" int hq_group_masked_gemm(const void* a, const void* b, const void* sfa, const void* sfb,
                                    const int32_t* masked_m, void* out, const void* bias, const float* alpha,
                                    int64_t num_experts, int64_t max_m_per_expert, int64_t n, int64_t k,
                                    int64_t sfa_bytes, int64_t sfb_bytes, int64_t ldo, int mode, int sm_count,
                                    int use_pdl, int device, void* stream, char* err, size_t errlen) {
    if (max_m_per_expert <= 0) {
        return hq::fail(err, errlen, HQ_ERR_INVALID, "max_m_per_expert must be greater than 0, got %lld",
                        (long long)max_m_per_expert);
    }
    return hq::grouped_gemm_impl(hq::kGroupMasked, a, b, sfa, sfb, out, bias, alpha, masked_m, num_experts,
                                 max_m_per_expert, num_experts * max_m_per_expert, n, k, sfa_bytes, sfb_bytes,
                                 ldo, mode, HQ_EPILOGUE_IDENTITY, nullptr, sm_count, use_pdl, device, stream, err, errlen);
}

extern "C" int hq_group_contiguous_gemm(const void* a, const void* b, const void* sfa, const void* sfb,
                                        const int32_t* expert_ids, void* out, const void* bias,
                                        const float* alpha, int64_t num_experts, int64_t m, int64_t n, int64_t k,
                                        int64_t sfa_bytes, int64_t sfb_bytes, int64_t ldo, int mode, int sm_count,
                                        int use_pdl, int device, void* stream, char* err, size_t errlen) {
    // the reference sizes its tiles by the mean rows per expert (csrc/kernel/gemm/group_contiguous_gemm.cu:80-87)
    const int64_t rows = num_experts > 0 ? m / num_experts : 0;
    if (num_experts > 0 && m > 0 && rows == 0) {
        return hq::no_group_tile(err, errlen, hq::kGroupContiguous, mode, rows, m, n, k);
    }
    return hq::grouped_gemm_impl(hq::kGroupContiguous, a, b, sfa, sfb, out, bias, alpha, expert_ids, num_experts,
                                 rows, m, n, k, sfa_bytes, sfb_bytes, ldo, mode, HQ_EPILOGUE_IDENTITY, nullptr, sm_count,
                                 use_pdl, device, stream, err, errlen);
}

extern "C" int hq_low_latency_gemm(const void* a, const void* b, const void* sfa, const void* sfb, void* out,
                                   const void* a2, const void* b2, const void* sfa2, const void* sfb2, void* out2,
                                   int64_t m, int64_t n, int64_t n2, int64_t k1, int64_t k2, int64_t sfa_stride,
                                   int64_t sfb_stride, int64_t sfa2_stride, int64_t sfb2_stride, int64_t ldo,
                                   int64_t ldo2, int use_sigmoid, int sm_count, int use_pdl, int device,
                                   void* stream, char* err, size_t errlen) {
    using hq::fail;
    const bool concat = a2 != nullptr;
    const bool dual = out2 != nullptr;
    const bool second_weight = b2 != nullptr;
    // same rules and texts as the reference's ResolveLlShapes (csrc/kernel/gemm/low_latency_utils.cuh:222-273)
    if ((a2 != nullptr) != (sfa2 != nullptr) || second_weight != (sfb2 != nullptr) || second_weight != (concat != dual)) {
        return fail(err, errlen, HQ_ERR_INVALID, "weight2 / sfb2 must come with either input2 / sfa2 or output2");
    }
    if (use_sigmoid && second_weight) {
        return fail(err, errlen, HQ_ERR_INVALID, "low_latency_mma_gemm use_sigmoid does not support input2 or output2");
    }
    if (m < 0 || n < 0 || n2 < 0 || k1 < 0 || k2 < 0 || n > INT32_MAX || n2 > INT32_MAX || k1 > INT32_MAX ||
        k2 > INT32_MAX) {
        return fail(err, errlen, HQ_ERR_INVALID, "problem sizes must be non-negative and below 2^31");
    }
    if (!dual) n2 = 0;
    if (!concat) k2 = 0;
    if (m > 16) return fail(err, errlen, HQ_ERR_INVALID, "low_latency_mma_gemm supports M <= 16, got M=%lld", (long long)m);
    if (n % 8 != 0 || n2 % 8 != 0) {
        return fail(err, errlen, HQ_ERR_INVALID, "low_latency_mma_gemm weight rows must be divisible by 8, got %lld and %lld",
                    (long long)n, (long long)n2);
    }
    if ((k1 + k2) % 256 != 0 || k1 % 128 != 0 || k2 % 128 != 0) {
        return fail(err, errlen, HQ_ERR_INVALID, "low_latency_mma_gemm K must be divisible by 256, got K=%lld",
                    (long long)(k1 + k2));
    }
    if (concat && k1 % 512 != 0) {
        return fail(err, errlen, HQ_ERR_INVALID, "concat-K K1 must be a multiple of 512, got K1=%lld", (long long)k1);
    }
    const int64_t kb2 = dual ? k1 / 32 : k2 / 32;  // scale columns of sfb2
    if (sfa_stride % 16 != 0 || sfb_stride % 16 != 0 || sfa_stride < k1 / 32 || sfb_stride < k1 / 32 ||
        (concat && (sfa2_stride % 16 != 0 || sfa2_stride < k2 / 32)) ||
        (second_weight && (sfb2_stride % 16 != 0 || sfb2_stride < kb2))) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "sfa / sfb / sfa2 / sfb2 must be plain row-major [rows, K / 32] scales "
                    "(group_wise_quant(..., use_swizzle=False)) with a row stride that is a multiple of 16 bytes; "
                    "got row strides %lld, %lld, %lld, %lld",
                    (long long)sfa_stride, (long long)sfb_stride, (long long)sfa2_stride, (long long)sfb2_stride);
    }
    if (m == 0 || (n == 0 && n2 == 0) || k1 + k2 == 0) return HQ_OK;
    const hq::DeviceGuard guard(device);
    if (!guard.ok()) return fail(err, errlen, HQ_ERR_CUDA, "cannot select CUDA device %d", device);
    const int sm_all = hq_sm_count(device);
    const int sm = sm_count > 0 ? (sm_count < sm_all || sm_all == 0 ? sm_count : sm_all) : sm_all;
    if (sm <= 0) return fail(err, errlen, HQ_ERR_CUDA, "cannot query the SM count of device %d", device);
    if (a == nullptr || b == nullptr || sfa == nullptr || sfb == nullptr || out == nullptr) {
        return fail(err, errlen, HQ_ERR_INVALID, "null pointer argument");
    }
    if (!hq::aligned(out, 16) || (dual && !hq::aligned(out2, 16)) || ldo % 8 != 0 || ldo < n ||
        (dual && (ldo2 % 8 != 0 || ldo2 < n2)) || !hq::aligned(sfa, 4) || !hq::aligned(sfb, 4) ||
        !hq::aligned(sfa2, 4) || !hq::aligned(sfb2, 4)) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "outputs must be 16-byte aligned with a row stride that is a multiple of 8 elements, scales "
                    "4-byte aligned");
    }

    using C = hq::Cfg<64, 0>;
    const int a_rows = int((m + 7) / 8 * 8);
    CUtensorMap tm_a, tm_b, tm_a2, tm_b2;
    const void* const a_tail = concat ? a2 : a;
    const int64_t k_tail = concat ? k2 : k1;
    const void* const b_other = second_weight ? b2 : b;
    const int64_t rows_other = dual ? n2 : n;
    const bool maps_ok =
        hq::make_tmap_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, a, uint64_t(k1), uint64_t(m), uint64_t(k1),
                         hq::kBKBytes, uint32_t(a_rows), CU_TENSOR_MAP_SWIZZLE_128B) &&
        hq::make_tmap_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, b, uint64_t(k1), uint64_t(n > 0 ? n : 8), uint64_t(k1),
                         hq::kBKBytes, 64, CU_TENSOR_MAP_SWIZZLE_128B) &&
        hq::make_tmap_2d(&tm_a2, CU_TENSOR_MAP_DATA_TYPE_UINT8, a_tail, uint64_t(k_tail), uint64_t(m), uint64_t(k_tail),
                         hq::kBKBytes, uint32_t(a_rows), CU_TENSOR_MAP_SWIZZLE_128B) &&
        hq::make_tmap_2d(&tm_b2, CU_TENSOR_MAP_DATA_TYPE_UINT8, b_other, uint64_t(k_tail), uint64_t(rows_other),
                         uint64_t(k_tail), hq::kBKBytes, 64, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!maps_ok) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "TMA descriptor encoding failed: input and weight must be 16-byte aligned, contiguous rows");
    }
    hq::LlParams p;
    p.sfa = static_cast<const uint8_t*>(sfa);
    p.sfb = static_cast<const uint8_t*>(sfb);
    p.sfa2 = static_cast<const uint8_t*>(concat ? sfa2 : sfa);
    p.sfb2 = static_cast<const uint8_t*>(second_weight ? sfb2 : sfb);
    p.sfa_stride = sfa_stride;
    p.sfb_stride = sfb_stride;
    p.sfa2_stride = concat ? sfa2_stride : sfa_stride;
    p.sfb2_stride = second_weight ? sfb2_stride : sfb_stride;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.out2 = static_cast<__nv_bfloat16*>(out2);
    p.ldo = ldo;
    p.ldo2 = ldo2;
    p.m = int(m);
    p.n = int(n);
    p.n2 = int(n2);
    p.k_tiles1 = int(k1 / hq::kBKBytes);
    p.k_tiles2 = int(k2 / hq::kBKBytes);
    p.a_rows = a_rows;
    p.sigmoid = use_sigmoid ? 1 : 0;

    static hq::SmemOptIn opt_in;
    HQ_CUDA_TRY(opt_in.ensure(hq::ll_gemm_kernel, hq::kLlSmemBytes));
    const int tiles = int((n + 63) / 64 + (n2 + 63) / 64);
    HQ_CUDA_TRY(hq::launch(hq::ll_gemm_kernel, dim3(std::min(sm, tiles)), dim3(hq::kLlThreads), size_t(hq::kLlSmemBytes),
                           static_cast<cudaStream_t>(stream), use_pdl != 0, 1, tm_a, tm_b, tm_a2, tm_b2, p));
    return HQ_OK;
}

extern "C" int hq_device_status(int device, void* stream, uint32_t* status, char* err, size_t errlen) {
    const hq::DeviceGuard guard(device);
    if (!guard.ok()) return hq::fail(err, errlen, HQ_ERR_CUDA, "cannot select CUDA device %d", device);
    HQ_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    uint32_t host[4] = {0, 0, 0, 0};
    HQ_CUDA_TRY(cudaMemcpyFromSymbol(host, hq::g_status, sizeof(host)));
    if (host[0] != 0) {
        const uint32_t zero[4] = {0, 0, 0, 0};
        HQ_CUDA_TRY(cudaMemcpyToSymbol(hq::g_status, zero, sizeof(zero)));
    }
    if (status != nullptr) *status = host[0];
    if (host[0] != 0) {
        return hq::fail(err, errlen, HQ_ERR_DEVICE,
                        "a GEMM role gave up on a bounded wait (status 0x%x: 1 producer, 2 MMA, 4 epilogue)",
                        host[0]);
    }
    return HQ_OK;
}

extern "C" int hq_selftest_bounded_wait(uint32_t limit_us, int device, void* stream, char* err, size_t errlen) {
    if (limit_us == 0 || limit_us > 100000u) {
        return hq::fail(err, errlen, HQ_ERR_INVALID, "limit_us must be in [1, 100000], got %u", limit_us);
    }
    const hq::DeviceGuard guard(device);
    if (!guard.ok()) return hq::fail(err, errlen, HQ_ERR_CUDA, "cannot select CUDA device %d", device);
    HQ_CUDA_TRY(hq::launch(hq::wait_selftest_kernel, dim3(1), dim3(64), size_t(0), static_cast<cudaStream_t>(stream),
                           false, 1, uint64_t(limit_us) * 1000ull));
    return HQ_OK;
}

extern "C" int hq_dense_gemm_allgather(const void* a, const void* b, const void* sfa, const void* sfb,
                                       void* const* outs, int world, int rank, int64_t m, int64_t n_local, int64_t k,
                                       int64_t sfa_bytes, int64_t sfb_bytes, int64_t ldo, int sm_count, int use_pdl,
                                       int device, void* stream, char* err, size_t errlen) {
    using hq::fail;
    if (world < 1 || world > 8 || rank < 0 || rank >= world || outs == nullptr) {
        return fail(err, errlen, HQ_ERR_INVALID, "world must be 1..8 with 0 <= rank < world and one output per rank, got "
                                                 "world=%d rank=%d", world, rank);
    }
    if (m < 1 || n_local < 1 || k < 1 || m > INT32_MAX || n_local * world > INT32_MAX || k > INT32_MAX) {
        return fail(err, errlen, HQ_ERR_INVALID, "input must be a 2D tensor of shape [M, K]");
    }
    if (n_local % 256 != 0 || k % 128 != 0 || m <= 128) {
        return fail(err, errlen, HQ_ERR_UNSUPPORTED,
                    "the fused all-gather runs on the 256x256 2-CTA tile: N per rank must be a multiple of 256, K of "
                    "128 and M > 128, got M=%lld N=%lld K=%lld", (long long)m, (long long)n_local, (long long)k);
    }
    const int64_t sf_k = k / 32;
    if (sfa_bytes < hq_sf_rows(m) * sf_k || sfb_bytes < hq_sf_rows(n_local) * sf_k) {
        return fail(err, errlen, HQ_ERR_INVALID, "sfa / sfb must hold whole 128-row SfAtoms");
    }
    if (ldo < n_local * world || ldo % 8 != 0) {
        return fail(err, errlen, HQ_ERR_INVALID, "the outputs are [M, world * N] matrices: row stride %lld is too small "
                                                 "or not a multiple of 8", (long long)ldo);
    }
    for (int r = 0; r < world; ++r) {
        if (outs[r] == nullptr || !hq::aligned(outs[r], 16)) {
            return fail(err, errlen, HQ_ERR_INVALID, "output %d is null or not 16-byte aligned", r);
        }
    }
    if (a == nullptr || b == nullptr || sfa == nullptr || sfb == nullptr || !hq::aligned(a, 16) || !hq::aligned(b, 16) ||
        !hq::aligned(sfa, 16) || !hq::aligned(sfb, 16)) {
        return fail(err, errlen, HQ_ERR_INVALID, "operands and scales must be non-null and 16-byte aligned");
    }
    const hq::DeviceGuard guard(device);
    if (!guard.ok()) return fail(err, errlen, HQ_ERR_CUDA, "cannot select CUDA device %d", device);
    const int sm_all = hq_sm_count(device);
    const int sm = sm_count > 0 ? (sm_count < sm_all || sm_all == 0 ? sm_count : sm_all) : sm_all;
    if (sm <= 0) return fail(err, errlen, HQ_ERR_CUDA, "cannot query the SM count of device %d", device);
    hq::GemmArgs g;
    g.a = a;
    g.b = b;
    g.sfa = static_cast<const uint8_t*>(sfa);
    g.sfb = static_cast<const uint8_t*>(sfb);
    g.alpha = nullptr;
    g.bias = nullptr;
    g.epi_op = HQ_EPILOGUE_IDENTITY;
    g.situ = hq::SituParams{};
    // this rank's own copy: columns [rank * n_local, (rank + 1) * n_local) of its [M, ldo] output
    g.out = static_cast<__nv_bfloat16*>(outs[rank]) + int64_t(rank) * n_local;
    g.ldo = ldo;
    g.m = int(m);
    g.n = int(n_local);
    g.grp = hq::GroupParams{hq::kGroupDense, 1, 0, nullptr};
    g.k_bytes = k;
    g.kq_dim = int(sf_k / 4);
    g.sm_count = sm;
    g.pdl = use_pdl != 0;
    g.direct_store = false;
    g.stream = static_cast<cudaStream_t>(stream);
    __nv_bfloat16* peers[8];
    int count = 0;
    for (int r = 0; r < world; ++r) {
        if (r != rank) peers[count++] = static_cast<__nv_bfloat16*>(outs[r]) + int64_t(rank) * n_local;
    }
    return hq::launch_pair<256, 0, true>(g, err, errlen, peers, count);
}

extern "C" int hq_dense_gemm_small_m_noalloc(const void* a, const void* b, const void* sfa, const void* sfb, void* out,
                                             int64_t m, int64_t n, int64_t k, int64_t sfa_bytes, int64_t sfb_bytes,
                                             int64_t ldo, int epilogue, int sm_count, int use_pdl, int device,
                                             void* stream, char* err, size_t errlen) {
    using hq::fail;
    if (epilogue != HQ_EPILOGUE_IDENTITY && epilogue != HQ_EPILOGUE_SIGMOID) {
        return fail(err, errlen, HQ_ERR_UNSUPPORTED, "Unsupported epilogue %d for w8a8-mxfp8", epilogue);
    }
    if (m < 0 || n < 0 || k < 0 || n > INT32_MAX || k > INT32_MAX) {
        return fail(err, errlen, HQ_ERR_INVALID, "input must be a 2D tensor of shape [M, K]");
    }
    if (m > hq::kNoAllocMaxM) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "hq_dense_gemm_small_m_noalloc takes at most %d activation rows (its scratch memory is a fixed "
                    "array), got M=%lld; use hq_dense_gemm", hq::kNoAllocMaxM, (long long)m);
    }
    if ((n + 127) / 128 > hq::kNoAllocMaxTiles) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "hq_dense_gemm_small_m_noalloc takes at most %d weight rows (one counter per 128 rows in a "
                    "fixed array), got N=%lld; use hq_dense_gemm", hq::kNoAllocMaxTiles * 128, (long long)n);
    }
    if (m == 0 || n == 0) return HQ_OK;
    if (k % 128 != 0 || n % 64 != 0 || k == 0) {
        return fail(err, errlen, HQ_ERR_INVALID, "No dense w8a8-mxfp8 tile for M=%lld (grid M=%lld), N=%lld, K=%lld",
                    (long long)m, (long long)m, (long long)n, (long long)k);
    }
    const int64_t sf_k = k / 32;
    if (sfa_bytes < hq_sf_rows(m) * sf_k || sfb_bytes < hq_sf_rows(n) * sf_k) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "sfa / sfb must hold whole 128-row SfAtoms: expected at least %lld and %lld elements, got %lld "
                    "and %lld", (long long)(hq_sf_rows(m) * sf_k), (long long)(hq_sf_rows(n) * sf_k),
                    (long long)sfa_bytes, (long long)sfb_bytes);
    }
    const hq::DeviceGuard guard(device);
    if (!guard.ok()) return fail(err, errlen, HQ_ERR_CUDA, "cannot select CUDA device %d", device);
    const int sm_all = hq_sm_count(device);
    const int sm = sm_count > 0 ? (sm_count < sm_all || sm_all == 0 ? sm_count : sm_all) : sm_all;
    if (sm <= 0) return fail(err, errlen, HQ_ERR_CUDA, "cannot query the SM count of device %d", device);
    if (a == nullptr || b == nullptr || sfa == nullptr || sfb == nullptr || out == nullptr) {
        return fail(err, errlen, HQ_ERR_INVALID, "null pointer argument");
    }
    if (!hq::aligned(a, 16) || !hq::aligned(b, 16) || !hq::aligned(sfa, 16) || !hq::aligned(sfb, 16) ||
        !hq::aligned(out, 16) || ldo < n || ldo % 8 != 0) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "operands, scales and output must be 16-byte aligned and the output row stride a "
                    "multiple of 8 elements");
    }
    // the same deal of the work as hq_dense_gemm makes for this shape, capped by the array's size
    hq::DecPlan plan = hq::decode_plan(m, n, k, sm);
    if (plan.ctas > hq::kNoAllocMaxCtas) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "hq_dense_gemm_small_m_noalloc runs on at most %d CTAs, this shape wants %d; pass a smaller sm_count",
                    hq::kNoAllocMaxCtas, plan.ctas);
    }
    hq::GemmArgs g;
    g.a = a;
    g.b = b;
    g.sfa = static_cast<const uint8_t*>(sfa);
    g.sfb = static_cast<const uint8_t*>(sfb);
    g.alpha = nullptr;
    g.bias = nullptr;
    g.epi_op = epilogue;
    g.situ = hq::SituParams{};
    g.out = static_cast<__nv_bfloat16*>(out);
    g.ldo = ldo;
    g.m = int(m);
    g.n = int(n);
    g.grp = hq::GroupParams{hq::kGroupDense, 1, 0, nullptr};
    g.k_bytes = k;
    g.kq_dim = int(sf_k / 4);
    g.sm_count = sm;
    g.pdl = use_pdl != 0;
    g.direct_store = false;
    g.stream = static_cast<cudaStream_t>(stream);
    return m <= 16 ? hq::launch_decode_noalloc<16>(g, plan, err, errlen) : hq::launch_decode_noalloc<32>(g, plan, err, errlen);
}

extern "C" int hq_selftest_decode_plan(int64_t n, int64_t k, int sm_count, int force_split, char* err,
                                       size_t errlen) {
    if (n < 1 || k < 128 || k % 128 != 0 || sm_count < 1) {
        return hq::fail(err, errlen, HQ_ERR_INVALID, "n >= 1, k a positive multiple of 128 and sm_count >= 1 expected");
    }
    hq::DecClusterLimits nominal = {};
    nominal.max_active[2] = 74;
    nominal.max_active[4] = 36;
    nominal.max_active[8] = 14;
    hq::DecPlan p = hq::dec_plan(int(n), k, sm_count, true, 16, force_split != 0, hq::decode_ring_bytes(16), &nominal);
    if (force_split == 2) {
        // the general even deal: every CTA one contiguous run of units, whatever the tile boundaries
        const int64_t units = int64_t(p.tiles) * p.ksteps;
        p.ctas = int(units < sm_count ? units : sm_count);
        p.aligned = 0;
        p.cluster = 0;
        p.fits32 = units * p.ctas < (int64_t(1) << 32) ? 1 : 0;
    }
    if (!hq::dec_plan_selfcheck(p)) {
        return hq::fail(err, errlen, HQ_ERR_INVALID, "unit deal inconsistent: tiles=%d ksteps=%d ctas=%d aligned=%d",
                        p.tiles, p.ksteps, p.ctas, p.aligned);
    }
    return HQ_OK;
}

extern "C" const char* hq_version(void) { return "halops_b200 0.1 (sm_100a)"; }
