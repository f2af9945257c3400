// Small-M ("decode") MXFP8 GEMM for sm_100a: out[M, N] = bf16(A[M, K] . B[N, K]^T), M <= 128.
//
// Included by gemm.cu inside namespace hq { namespace { ... } }, after the barrier, wait and
// tensor-map helpers.  Replaces the reference's operand-swapped small-M tiles
// (csrc/kernel/gemm/gemm_kernel.cuh:499-547, gemm_tile.cuh:203-216, epilogue.cuh:377-711).
//
// The weight streams through once, so the kernel is bound by HBM, not by the tensor cores;
// what has to be kept small is everything else: the work of the thread that issues the MMAs
// (about 90 cycles per tcgen05.mma and 230 per tcgen05.commit whatever their size) and the
// epilogue.  Design:
//   * Operands are swapped: 128 weight rows are the M of tcgen05.mma, the activations its
//     N (16 / 32 / 64 / 128 columns).  One instruction then consumes 4 KB of weights instead
//     of the 2 KB of a 128 x 64 tile with the activations as M.
//   * A stage holds 256 bytes of K per row (two 128-byte-swizzled boxes per operand): half
//     as many barrier round trips and commits per byte of weight.
//   * Two threads issue the MMAs of alternate k-steps into accumulators of their own, so
//     they need no hand-over; the epilogue adds the two accumulators.  One thread alone
//     needs about 1000 cycles per 32 KB step (33 bytes per cycle and CTA), less than an SM's
//     share of HBM when fewer CTAs than SMs have work.
//   * Work is cut into units of (128 weight rows) x (256 bytes of K).  Normally a CTA works
//     whole tiles.  When there are too few tiles to keep HBM busy, the units are dealt out
//     evenly over the CTAs in one contiguous run each ("stream-K"), and a tile whose K range
//     is shared by several CTAs is summed through float32 partial tiles in a global scratch
//     buffer: every contributor stores its partial tile and counts itself on the tile's
//     counter; the last one to arrive adds the partial tiles in K order (not arrival order,
//     so the result is deterministic) and stores the bf16 result.  No CTA waits for another.
//   * The accumulator is [128 weight rows (lanes)] x [activations (columns)]: the epilogue
//     transposes 16 columns at a time through a small shared-memory buffer per warp and
//     stores a [16 rows x 32 columns] box of the output with one TMA store, which also clips
//     rows past M and columns past N.
//
// Warps: 0 loader, 1 and 7 MMA issuers (warp 1 allocates tensor memory), 2-5 epilogue,
// 6 scale copies (tcgen05.cp, a few k-steps ahead of the MMAs).

constexpr int kDecThreads = 256;
constexpr int kDecRows = 128;      // weight rows per tile (the M of the MMA)
constexpr int kDecStepBytes = 256; // bytes of K per stage row
constexpr int kDecIssuers = 2;     // threads issuing MMAs, each into its own accumulator
constexpr int kDecEpiBufBytes = 16 * 64;  // staging of one [16 rows x 32 columns] bf16 box
constexpr int kDecCounterSlots = 65536;   // tiles a launch may have (counters in the scratch buffer)

template <int NACT>
struct DecCfg {
    static_assert(NACT == 16 || NACT == 32 || NACT == 64 || NACT == 128, "activation widths built");
    static constexpr int kWBytes = kDecRows * kDecStepBytes;  // two boxes of 128 rows x 128 bytes
    static constexpr int kXBytes = NACT * kDecStepBytes;      // two boxes of NACT rows x 128 bytes
    static constexpr int kSfBytes = 2 * 512;                  // per operand: the SfAtoms of two k-tiles
    static constexpr int kStageBytes = kWBytes + kXBytes + 2 * kSfBytes;
    static constexpr int kEpiBytes = kEpiWarps * 2 * kDecEpiBufBytes;
    static constexpr int kBarBytes = 1024;
    static constexpr int kStagesFit = (kSmemBudget - kEpiBytes - kBarBytes - 1024) / kStageBytes;
    static constexpr int kStages = kStagesFit > 8 ? 8 : kStagesFit;
    static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + kBarBytes + 1024;
    // Tensor memory: kAccStages accumulator stages of kDecIssuers x NACT fp32 columns (one
    // stage for the widest activations: two would not fit beside the scales), then kSfSets
    // sets of 16 scale columns (weights: 2 atoms x 4 columns, activations: 2 x 4).  A set is
    // reused once the MMAs that read it have released their stage, which the copy thread can
    // only tell apart from a later release of the same stage when there are no more sets than
    // stages.
    static constexpr int kAccStages = NACT == 128 ? 1 : 2;
    static constexpr int kSfSets = kStages < 4 ? kStages : 4;
    static constexpr int kSfCol0 = kAccStages * kDecIssuers * NACT;
    static constexpr int kColsUsed = kSfCol0 + kSfSets * 16;
    static constexpr int kTmemCols = kColsUsed <= 32 ? 32 : kColsUsed <= 64 ? 64 : kColsUsed <= 128 ? 128
                                     : kColsUsed <= 256 ? 256 : 512;
    static_assert(kStages >= 2 && kColsUsed <= 512, "shared / tensor memory budget");
};

// How the (tile, k-step) units are dealt out: CTA c works the units [begin(c), begin(c + 1)).
// `aligned` keeps the runs on tile boundaries (no partial tiles, no scratch traffic).
struct DecPlan {
    int tiles;    // 128-row weight tiles
    int ksteps;   // 256-byte steps of K (the last may hold 128 bytes)
    int ctas;
    int aligned;
    int fits32;   // units * ctas < 2^32: the device may deal in 32-bit arithmetic
    int cluster;  // > 1: the CTAs of one tile form a thread-block cluster of this size and exchange
                  // their partial tiles through shared memory instead of the scratch buffer
};

__host__ __device__ inline int64_t dec_begin(const DecPlan& p, int c) {
    if (p.aligned) return int64_t(uint32_t(c) * uint32_t(p.tiles) / uint32_t(p.ctas)) * p.ksteps;  // ctas, tiles <= 65536
    // (32-bit division is several times cheaper on the device; fits32: units * ctas < 2^32)
    if (p.fits32) return int64_t(uint32_t(c) * (uint32_t(p.tiles) * uint32_t(p.ksteps)) / uint32_t(p.ctas));
    return int64_t(c) * p.tiles * p.ksteps / p.ctas;
}
// The CTA whose run holds unit u: the largest c with begin(c) <= u.
__host__ __device__ inline int dec_owner(const DecPlan& p, int64_t u) {
    if (p.aligned) return int(((u / p.ksteps + 1) * p.ctas - 1) / p.tiles);
    if (p.fits32) return int(((uint32_t(u) + 1u) * uint32_t(p.ctas) - 1u) / (uint32_t(p.tiles) * uint32_t(p.ksteps)));
    return int(((u + 1) * p.ctas - 1) / (int64_t(p.tiles) * p.ksteps));
}

// One piece of a CTA's run: k-steps [k0, k1) of one tile.
struct DecSeg {
    int tile, k0, k1;
    bool partial;  // other CTAs hold the rest of this tile's K
};
struct DecWalk {
    DecPlan p;
    int64_t u, end;
    __host__ __device__ DecWalk(const DecPlan& plan, int c) : p(plan), u(dec_begin(plan, c)), end(dec_begin(plan, c + 1)) {}
    __host__ __device__ bool next(DecSeg& s) {
        if (u >= end) return false;
        if (p.aligned) {
            // runs of whole tiles: 32-bit arithmetic on the way to the first load
            s.tile = int(uint32_t(u) / uint32_t(p.ksteps));
            s.k0 = 0;
            s.k1 = p.ksteps;
            s.partial = false;
            u += p.ksteps;
            return true;
        }
        s.tile = p.fits32 ? int(uint32_t(u) / uint32_t(p.ksteps)) : int(u / p.ksteps);
        s.k0 = int(u - int64_t(s.tile) * p.ksteps);
        const int64_t left = end - u;
        s.k1 = left < p.ksteps - s.k0 ? s.k0 + int(left) : p.ksteps;
        s.partial = s.k0 != 0 || s.k1 != p.ksteps;
        u += s.k1 - s.k0;
        return true;
    }
};
// Scratch slot of CTA c's partial sums for `tile`: slot 0 when its run begins inside (or at
// the start of) the tile, slot 1 when it began earlier and ends in it.  A run touches at most
// one tile of each kind.
__host__ __device__ inline int dec_slot(const DecPlan& p, int c, int tile) {
    return c * 2 + (dec_begin(p, c) >= int64_t(tile) * p.ksteps ? 0 : 1);
}

struct DecParams {
    const uint8_t* sfw;   // weight scales (SfAtom order, N rounded up to 128 rows)
    const uint8_t* sfx;   // activation scales (SfAtom order, one 128-row atom row)
    float* scratch;       // [ctas * 2][NACT][128] float32 partial tiles
    int* counters;        // [tiles], zero between launches
    int m, n;
    int64_t k_bytes;
    int kq_dim;           // SfAtoms along K
    int x_rows;           // rows of the activation box (m rounded up to 8)
    int epi_op;
    int early_weights;    // the weight and its scales are read before the preceding kernel is known to be complete
    DecPlan plan;
};

__device__ __forceinline__ void tc_load_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// Rendezvous of the four epilogue warps on an mbarrier (one arrival per warp): unlike bar.sync
// the wait is bounded and gives up when the CTA aborts.  Shared-memory writes before it are
// visible after it (release / acquire at CTA scope).
__device__ __forceinline__ bool epi_rendezvous(Barriers* bars, uint32_t& phase, int lane, volatile uint32_t* abort) {
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars->epi_sync));
    const bool ok = wait_bar(ptx::smem_u32(&bars->epi_sync), phase & 1u, abort, kStatusEpilogue);
    ++phase;
    return ok;
}

// Bounded wait on a barrier that CTAs of the cluster arrive on with release semantics: acquires
// what they wrote into this CTA's shared memory before arriving.
__device__ __forceinline__ bool wait_bar_cluster(uint32_t bar, uint32_t parity, volatile uint32_t* abort, uint32_t code) {
    if (ptx::mbar_try_wait_cluster(bar, parity)) return true;
    const uint64_t t0 = ptx::globaltimer_ns();
    uint32_t spins = 0;
    while (!ptx::mbar_try_wait_cluster(bar, parity)) {
        if ((++spins & 31u) == 0u) {
            if (*abort != 0u) return false;
            if (ptx::globaltimer_ns() - t0 > kTimeoutNs) {
                *abort = 1u;
                atomicOr(&g_status[0], code);
                return false;
            }
        }
    }
    return true;
}

// bf16(y) or bf16(sigmoid(y)) in the reference's formulation (see epilogue_chunk), as 16 bits
__device__ __forceinline__ uint16_t dec_finish(float y, int epi_op) {
    if (epi_op == HQ_EPILOGUE_SIGMOID) y = fmaf(0.5f, tanh_fast(0.5f * y), 0.5f);
    return __bfloat16_as_ushort(__float2bfloat16_rn(y));
}

// Output rows [row0, row0 + 16) x columns [col0, col0 + 32) from the 16 values every lane
// holds (lane = column, v[j] = row row0 + j): transposed through `buf`, stored by TMA.
__device__ __forceinline__ void dec_store_box(const CUtensorMap* tm_o, uint32_t buf, int lane, const float (&v)[16],
                                              int epi_op, int col0, int row0) {
    // the TMA store that last read this buffer (two stores ago) must be done with it
    if (lane == 0) ptx::bulk_wait_read<1>();
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        asm volatile("st.shared.b16 [%0], %1;" ::"r"(buf + j * 64 + lane * 2), "h"(dec_finish(v[j], epi_op)) : "memory");
    }
    ptx::fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
        ptx::tma_store_2d(tm_o, buf, col0, row0);
        ptx::bulk_commit();
    }
}

template <int NACT>
__global__ void __launch_bounds__(kDecThreads, 1)
gemm_decode_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                   const __grid_constant__ CUtensorMap tm_o, const DecParams p) {
    using C = DecCfg<NACT>;
    // the descriptors come from global memory: ask for them before anything else (each request
    // holds its thread for a few hundred cycles, so the loader's thread asks only for the one it
    // needs first)
    if (threadIdx.x == 0) ptx::prefetch_tmap(&tm_w);
    if (threadIdx.x == 64) {
        ptx::prefetch_tmap(&tm_x);
        ptx::prefetch_tmap(&tm_o);
    }
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* const smem = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
    const uint32_t w_base = smem_base;
    const uint32_t x_base = w_base + C::kStages * C::kWBytes;
    const uint32_t sfw_base = x_base + C::kStages * C::kXBytes;
    const uint32_t sfx_base = sfw_base + C::kStages * C::kSfBytes;
    const uint32_t epi_base = sfx_base + C::kStages * C::kSfBytes;
    Barriers* const bars = reinterpret_cast<Barriers*>(smem + C::kStages * C::kStageBytes + C::kEpiBytes);
    static_assert(sizeof(Barriers) <= C::kBarBytes, "barrier block");
    volatile uint32_t* const abort = &bars->abort;
    __shared__ int s_last;  // epilogue: this CTA is the last contributor of the tile at hand

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int cta = blockIdx.x;
    const int k_tiles = int(p.k_bytes / kBKBytes);  // 128-byte k-tiles; a k-step holds two, the last maybe one

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&bars->full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&bars->empty[s]), 1);
        }
        for (int s = 0; s < C::kAccStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&bars->acc_full[s]), kDecIssuers);
            ptx::mbar_init(ptx::smem_u32(&bars->acc_empty[s]), kEpiWarps);
        }
        for (int s = 0; s < C::kSfSets; ++s) ptx::mbar_init(ptx::smem_u32(&bars->sf_ready[s]), 1);
        ptx::mbar_init(ptx::smem_u32(&bars->epi_sync), kEpiWarps);
        if (p.plan.cluster > 1) {
            ptx::mbar_init(ptx::smem_u32(&bars->turn[0]), 1);  // "the first CTA's ring is free"
            ptx::mbar_init(ptx::smem_u32(&bars->recv_full), uint32_t(p.plan.cluster - 1) * kEpiWarps);
        }
        bars->abort = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc<1>(ptx::smem_u32(&bars->tmem_base), C::kTmemCols);
        ptx::tmem_relinquish<1>();
    }
    ptx::tc_fence_before();
    __syncthreads();
    // the other CTAs' barriers exist before anyone signals across the cluster
    if (p.plan.cluster > 1) ptx::cluster_sync();
    ptx::tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    // Nothing below may read what the previous kernel wrote before this returns.  With
    // early_weights only the loader waits, after it has asked for the weight of its first ring
    // of stages: the caller vouches that the weight and its scales are not written by the
    // preceding kernel.  The other roles touch global memory only behind barriers that the
    // loader's later copies (the activation) complete, so they run after its wait as well.
    if (p.early_weights == 0) ptx::pdl_wait();

    if (warp == 0) {
        // ------------------------------------------------------------ loader
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            const auto arm = [&](uint32_t s, int boxes) {
                ptx::mbar_arrive_expect_tx(ptx::smem_u32(&bars->full[s]),
                                           uint32_t(boxes) * (kDecRows * kBKBytes + p.x_rows * kBKBytes + 1024));
            };
            const auto load_weight = [&](uint32_t s, int boxes, int ks, int tile) {
                const uint32_t full = ptx::smem_u32(&bars->full[s]);
                for (int b = 0; b < boxes; ++b) {
                    ptx::tma_load_2d(w_base + s * C::kWBytes + b * (kDecRows * kBKBytes), &tm_w,
                                     ks * kDecStepBytes + b * kBKBytes, tile * kDecRows, full);
                }
            };
            const auto load_weight_scales = [&](uint32_t s, int boxes, int ks, int tile) {
                ptx::bulk_load(sfw_base + s * C::kSfBytes, p.sfw + int64_t(tile) * p.kq_dim * 512 + int64_t(ks) * 1024,
                               uint32_t(boxes) * 512, ptx::smem_u32(&bars->full[s]));
            };
            if (p.early_weights != 0) {
                // the first ring of stages: every stage is free, its barrier is armed for all
                // the bytes of the step, and the weight's share is asked for now
                DecWalk ahead(p.plan, cta);
                DecSeg as;
                uint32_t pre = 0;
                while (pre < uint32_t(C::kStages) && ahead.next(as)) {
                    for (int ks = as.k0; ks < as.k1 && pre < uint32_t(C::kStages); ++ks, ++pre) {
                        const int boxes = min(2, k_tiles - 2 * ks);
                        arm(pre, boxes);
                        load_weight(pre, boxes, ks, as.tile);
                        load_weight_scales(pre, boxes, ks, as.tile);
                    }
                }
                // (letting the next kernel of the stream start here already, before this one's wait,
                // measured slower: 7.5 against 7.0 us per GEMM in a chain of 8 x 7168 x 2048)
                ptx::pdl_wait();
            }
            DecWalk walk(p.plan, cta);
            DecSeg sg;
            while (ok && walk.next(sg)) {
                for (int ks = sg.k0; ks < sg.k1; ++ks, ++it) {
                    const uint32_t s = it % C::kStages;
                    const int boxes = min(2, k_tiles - 2 * ks);  // 128-byte k-tiles in this step
                    const bool asked = p.early_weights != 0 && it < uint32_t(C::kStages);
                    if (!asked) {
                        ok = wait_bar(ptx::smem_u32(&bars->empty[s]), ((it / C::kStages) & 1u) ^ 1u, abort,
                                      kStatusProducer);
                        if (!ok) break;
                        arm(s, boxes);
                        // the weight first: it is what the step waits for
                        load_weight(s, boxes, ks, sg.tile);
                    }
                    const uint32_t full = ptx::smem_u32(&bars->full[s]);
                    for (int b = 0; b < boxes; ++b) {
                        ptx::tma_load_2d(x_base + s * C::kXBytes + b * (NACT * kBKBytes), &tm_x,
                                         ks * kDecStepBytes + b * kBKBytes, 0, full);
                    }
                    if (!asked) load_weight_scales(s, boxes, ks, sg.tile);
                    ptx::bulk_load(sfx_base + s * C::kSfBytes, p.sfx + int64_t(ks) * 1024, uint32_t(boxes) * 512, full);
                }
            }
            ptx::pdl_launch_dependents();
        }
    } else if (warp == 6) {
        // ------------------------------------------------------------ scale copies: shared -> tensor memory
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            DecWalk walk(p.plan, cta);
            DecSeg sg;
            while (ok && walk.next(sg)) {
                for (int ks = sg.k0; ks < sg.k1; ++ks, ++it) {
                    const uint32_t s = it % C::kStages;
                    ok = wait_bar(ptx::smem_u32(&bars->full[s]), (it / C::kStages) & 1u, abort, kStatusProducer);
                    if (ok && it >= uint32_t(C::kSfSets)) {
                        // the MMAs of step it - kSfSets read this set: done once they released their stage
                        const uint32_t prev = it - uint32_t(C::kSfSets);
                        ok = wait_bar(ptx::smem_u32(&bars->empty[prev % C::kStages]), (prev / C::kStages) & 1u, abort,
                                      kStatusProducer);
                    }
                    if (!ok) break;
                    ptx::tc_fence_after();
                    const uint32_t set = tmem + C::kSfCol0 + (it % C::kSfSets) * 16;
                    const int boxes = min(2, k_tiles - 2 * ks);
                    for (int b = 0; b < boxes; ++b) {
                        ptx::tc_copy_sf<1>(set + b * 4, ptx::smem_desc(sfw_base + s * C::kSfBytes + b * 512, 0, 128, 0));
                        ptx::tc_copy_sf<1>(set + 8 + b * 4, ptx::smem_desc(sfx_base + s * C::kSfBytes + b * 512, 0, 128, 0));
                    }
                    ptx::tc_commit(ptx::smem_u32(&bars->sf_ready[it % C::kSfSets]));
                }
            }
        }
    } else if (warp == 1 || warp == 7) {
        // ------------------------------------------------------------ MMA issuers
        // Issuer `me` takes the k-steps of a piece whose index inside the piece is me modulo
        // kDecIssuers and accumulates them in its own columns; nothing orders the two threads.
        if (lane == 0) {
            const int me = warp == 1 ? 0 : 1;
            uint32_t it = 0;
            uint32_t t = 0;
            bool ok = true;
            DecWalk walk(p.plan, cta);
            DecSeg sg;
            for (; ok && walk.next(sg); ++t) {
                const uint32_t as = t % C::kAccStages;
                // both issuers wait for the drained stage, also the one that may have nothing to
                // issue in a one-step piece: its arrival below must not run ahead of the stage's
                // previous use
                ok = wait_bar(ptx::smem_u32(&bars->acc_empty[as]), ((t / C::kAccStages) & 1u) ^ 1u, abort, kStatusMma);
                if (!ok) break;
                ptx::tc_fence_after();
                const uint32_t acc = tmem + (as * kDecIssuers + me) * NACT;
                bool issued = false;
                for (int ks = sg.k0; ks < sg.k1; ++ks, ++it) {
                    if (((ks - sg.k0) & (kDecIssuers - 1)) != me) continue;
                    const uint32_t s = it % C::kStages;
                    // scales in tensor memory (the copy thread waited for the stage before it
                    // copied); the stage's own barrier orders this thread after the TMA writes
                    ok = wait_bar(ptx::smem_u32(&bars->sf_ready[it % C::kSfSets]), (it / C::kSfSets) & 1u, abort,
                                  kStatusMma) &&
                         wait_bar(ptx::smem_u32(&bars->full[s]), (it / C::kStages) & 1u, abort, kStatusMma);
                    if (!ok) break;
                    ptx::tc_fence_after();
                    const uint32_t set = tmem + C::kSfCol0 + (it % C::kSfSets) * 16;
                    const int boxes = min(2, k_tiles - 2 * ks);
                    for (int b = 0; b < boxes; ++b) {
                        const uint64_t wdesc = ptx::smem_desc(w_base + s * C::kWBytes + b * (kDecRows * kBKBytes), 16, 1024, 2);
                        const uint64_t xdesc = ptx::smem_desc(x_base + s * C::kXBytes + b * (NACT * kBKBytes), 16, 1024, 2);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            // the weights are the instruction's A (128 rows), the activations its B
                            ptx::tc_mma_block_scaled<1, 0>(acc, wdesc + uint64_t(k * 2), xdesc + uint64_t(k * 2),
                                                           instr_desc<NACT, 0>(uint32_t(k)), set + b * 4,
                                                           set + 8 + b * 4, (issued || b > 0 || k > 0) ? 1u : 0u);
                        }
                    }
                    issued = true;
                    ptx::tc_commit(ptx::smem_u32(&bars->empty[s]));
                }
                if (!ok) break;
                // a commit tracks the executing thread's operations: each issuer reports its own
                if (issued) {
                    ptx::tc_commit(ptx::smem_u32(&bars->acc_full[as]));
                } else {
                    ptx::mbar_arrive(ptx::smem_u32(&bars->acc_full[as]));
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2-5)
        const uint32_t lane_base = (warp & 3) * 32;  // tensor-memory lanes this warp may read
        const int row = int(lane_base) + lane;      // weight row of this thread inside the tile
        const int tid = (warp - 2) * 32 + lane;
        const uint32_t my_bufs = epi_base + (warp - 2) * 2 * kDecEpiBufBytes;
        const int m_chunks = (min(p.m, NACT) + 15) / 16;  // 16-column chunks that hold rows of the output
        uint32_t t = 0;
        uint32_t stores = 0;
        uint32_t sync_phase = 0;
        bool ok = true;
        DecWalk walk(p.plan, cta);
        DecSeg sg;
        for (; ok && walk.next(sg); ++t) {
            const uint32_t as = t % C::kAccStages;
            ok = wait_bar(ptx::smem_u32(&bars->acc_full[as]), (t / C::kAccStages) & 1u, abort, kStatusEpilogue);
            if (!ok) break;
            ptx::tc_fence_after();
            const uint32_t acc = tmem + as * kDecIssuers * NACT + (lane_base << 16);
            const bool two = sg.k1 - sg.k0 > 1;  // the second issuer had steps of this piece
            const int col0 = sg.tile * kDecRows + int(lane_base);  // first output column of this warp
            if (sg.partial && p.plan.cluster > 1) {
                // ---- the tile's CTAs are one cluster: partial tiles go into the first CTA's shared
                // memory (its operand ring, idle once its MMAs have completed), which adds them in
                // rank order, i.e. in K order, and stores the result
                const uint32_t crank = ptx::cluster_ctarank();
                const uint32_t ring_ok = ptx::smem_u32(&bars->turn[0]);
                const uint32_t recv_full = ptx::smem_u32(&bars->recv_full);
                constexpr uint32_t kPartBytes = NACT * kDecRows * 4;
                if (crank != 0) {
                    ok = wait_bar_cluster(ring_ok, 0, abort, kStatusEpilogue);
                    if (!ok) break;
                    const uint32_t dst = ptx::mapa_cluster(w_base, 0) + (crank - 1) * kPartBytes + uint32_t(row) * 4;
#pragma unroll 1
                    for (int ci = 0; ci < m_chunks; ++ci) {
                        uint32_t r0[16], r1[16];
                        tc_load_32x16(acc + ci * 16, r0);
                        if (two) tc_load_32x16(acc + NACT + ci * 16, r1);
                        ptx::tc_wait_ld();
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float v = two ? __uint_as_float(r0[j]) + __uint_as_float(r1[j]) : __uint_as_float(r0[j]);
                            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(dst + (ci * 16 + j) * (kDecRows * 4)), "f"(v)
                                         : "memory");
                        }
                    }
                    ptx::tc_fence_before();
                    // every lane's stores are ordered before the warp's one remote arrival
                    __syncwarp();
                    if (lane == 0) {
                        ptx::mbar_arrive(ptx::smem_u32(&bars->acc_empty[as]));
                        ptx::mbar_arrive_cluster_addr(ptx::mapa_cluster(recv_full, 0));
                    }
                } else {
                    // acc_full has completed: this CTA's MMAs no longer read the ring
                    if (tid == 0) {
                        for (int r = 1; r < p.plan.cluster; ++r) ptx::mbar_arrive_cluster_addr(ptx::mapa_cluster(ring_ok, uint32_t(r)));
                    }
                    ok = wait_bar_cluster(recv_full, 0, abort, kStatusEpilogue);
                    if (!ok) break;
#pragma unroll 1
                    for (int ci = 0; ci < m_chunks; ++ci) {
                        uint32_t r0[16], r1[16];
                        tc_load_32x16(acc + ci * 16, r0);
                        if (two) tc_load_32x16(acc + NACT + ci * 16, r1);
                        ptx::tc_wait_ld();
                        float v[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = two ? __uint_as_float(r0[j]) + __uint_as_float(r1[j]) : __uint_as_float(r0[j]);
                        for (int r = 1; r < p.plan.cluster; ++r) {
                            const uint32_t src = w_base + uint32_t(r - 1) * kPartBytes + uint32_t(row) * 4 + ci * 16 * (kDecRows * 4);
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                float x;
                                asm volatile("ld.shared.f32 %0, [%1];" : "=f"(x) : "r"(src + j * (kDecRows * 4)));
                                v[j] += x;
                            }
                        }
                        dec_store_box(&tm_o, my_bufs + (stores & 1u) * kDecEpiBufBytes, lane, v, p.epi_op, col0, ci * 16);
                        ++stores;
                    }
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars->acc_empty[as]));
                }
                continue;
            }
            float* const mine = !sg.partial ? nullptr
                                : p.scratch + int64_t(dec_slot(p.plan, cta, sg.tile)) * (NACT * kDecRows) + row;
#pragma unroll 1
            for (int ci = 0; ci < m_chunks; ++ci) {
                uint32_t r0[16], r1[16];
                tc_load_32x16(acc + ci * 16, r0);
                if (two) tc_load_32x16(acc + NACT + ci * 16, r1);
                ptx::tc_wait_ld();
                if (ci == m_chunks - 1) {
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars->acc_empty[as]));
                }
                float v[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = two ? __uint_as_float(r0[j]) + __uint_as_float(r1[j]) : __uint_as_float(r0[j]);
                if (!sg.partial) {
                    dec_store_box(&tm_o, my_bufs + (stores & 1u) * kDecEpiBufBytes, lane, v, p.epi_op, col0, ci * 16);
                    ++stores;
                } else {
                    // this CTA holds only part of the tile's K: float32 partial tile to the scratch buffer
#pragma unroll
                    for (int j = 0; j < 16; ++j) __stcg(mine + (ci * 16 + j) * kDecRows, v[j]);
                }
            }
            if (!sg.partial) continue;
            // every thread's stores are visible device-wide before the CTA counts itself
            __threadfence();
            if (!(ok = epi_rendezvous(bars, sync_phase, lane, abort))) break;
            const int64_t u0 = int64_t(sg.tile) * p.plan.ksteps;
            const int first = dec_owner(p.plan, u0);
            const int parts = dec_owner(p.plan, u0 + p.plan.ksteps - 1) - first + 1;
            if (tid == 0) {
                const int prev = atomicAdd(p.counters + sg.tile, 1);
                s_last = prev == parts - 1 ? 1 : 0;
                if (prev == parts - 1) p.counters[sg.tile] = 0;  // ready for the next launch
            }
            if (!(ok = epi_rendezvous(bars, sync_phase, lane, abort))) break;
            const bool last = s_last != 0;
            // s_last may be rewritten for the next tile only after everyone has read it
            if (!(ok = epi_rendezvous(bars, sync_phase, lane, abort))) break;
            if (!last) continue;
            __threadfence();
            // the last contributor adds the partial tiles in K order and stores the result; the
            // loads of up to four partial tiles are in flight together
            const float* src[4];
#pragma unroll 1
            for (int ci = 0; ci < m_chunks; ++ci) {
                float sum[16];
                for (int q0 = 0; q0 < parts; q0 += 4) {
                    float v[4][16];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int qq = min(q0 + q, parts - 1);
                        src[q] = p.scratch + int64_t(dec_slot(p.plan, first + qq, sg.tile)) * (NACT * kDecRows) + row +
                                 ci * 16 * kDecRows;
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[q][j] = __ldcg(src[q] + j * kDecRows);
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        if (q0 + q < parts) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) sum[j] = (q0 + q == 0) ? v[q][j] : sum[j] + v[q][j];
                        }
                    }
                }
                dec_store_box(&tm_o, my_bufs + (stores & 1u) * kDecEpiBufBytes, lane, sum, p.epi_op, col0, ci * 16);
                ++stores;
            }
        }
        // the staging buffers must outlive the stores that read them
        if (lane == 0) ptx::bulk_wait_read<0>();
    }

    if (*abort != 0u) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before();
    __syncthreads();
    // no CTA of a cluster leaves while another may still write into its shared memory or
    // arrive on its barriers (every wait above is bounded, so all of them get here)
    if (p.plan.cluster > 1) ptx::cluster_sync();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc<1>(tmem, C::kTmemCols);
    }
}

// ---------------------------------------------------------------------------- host side

// Scratch of the decode kernel: partial tiles and tile counters, one buffer per (device, stream)
// so that launches on different streams never share it.  Allocated on first use (with
// cudaMalloc: the first decode-sized call on a stream should come before any stream capture)
// and kept until the process ends.
struct DecScratch {
    float* partials = nullptr;
    int* counters = nullptr;
};
constexpr size_t kDecPartialBytes = size_t(2) * 160 * 128 * kDecRows * sizeof(float);  // up to 160 CTAs, NACT = 128
constexpr size_t kDecScratchBytes = kDecPartialBytes + size_t(kDecCounterSlots) * sizeof(int);

inline bool dec_scratch(int dev, cudaStream_t stream, DecScratch* out) {
    struct Entry {
        int dev;
        cudaStream_t stream;
        DecScratch s;
    };
    static std::mutex mu;
    static Entry entries[64];
    static int count = 0;
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < count; ++i) {
        if (entries[i].dev == dev && entries[i].stream == stream) {
            *out = entries[i].s;
            return true;
        }
    }
    if (count == 64) return false;  // the caller falls back to runs on tile boundaries (no scratch)
    void* base = nullptr;
    if (cudaMalloc(&base, kDecScratchBytes) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    if (cudaMemset(static_cast<uint8_t*>(base) + kDecPartialBytes, 0, size_t(kDecCounterSlots) * sizeof(int)) !=
        cudaSuccess) {
        cudaFree(base);
        return false;
    }
    entries[count].dev = dev;
    entries[count].stream = stream;
    entries[count].s.partials = static_cast<float*>(base);
    entries[count].s.counters = reinterpret_cast<int*>(static_cast<uint8_t*>(base) + kDecPartialBytes);
    *out = entries[count].s;
    ++count;
    return true;
}

// Deal of the units.  Whole tiles per CTA unless the weight has so few tiles that the CTAs at
// work cannot keep HBM busy and the float32 exchange of partial tiles at the end of a split
// run costs less than it saves.  A split deals every tile to `s` CTAs (s a power of two with
// tiles * s <= SMs).
struct DecClusterLimits {
    int max_active[9];  // clusters of 2, 4, 8 CTAs of this kernel that can be resident at once
};

inline DecPlan dec_plan(int n, int64_t k_bytes, int sm_count, bool allow_split, int nact, bool force_split,
                        int64_t ring_bytes, const DecClusterLimits* clusters) {
    DecPlan p;
    p.tiles = (n + kDecRows - 1) / kDecRows;
    p.ksteps = int((k_bytes + kDecStepBytes - 1) / kDecStepBytes);
    p.fits32 = 0;
    p.cluster = 0;
    const int whole_ctas = p.tiles < sm_count ? p.tiles : sm_count;
    p.ctas = whole_ctas;
    p.aligned = 1;
    int s = 1;
    while (p.tiles * s * 2 <= sm_count && s * 2 <= p.ksteps) s *= 2;
    if (!allow_split || s == 1 || p.tiles > kDecCounterSlots || p.tiles * s > 160) return p;
    // A cluster (at most 8 CTAs, the portable maximum) exchanges the partial tiles through the
    // first CTA's shared memory, if they fit into its operand ring and all of the tiles' clusters
    // can be resident at once (a second wave of clusters would wait for the whole first one).
    int sc = 0;
    if (clusters != nullptr) {
        sc = s > 8 ? 8 : s;
        while (sc > 1 && (int64_t(sc - 1) * nact * kDecRows * 4 > ring_bytes || p.tiles > clusters->max_active[sc])) sc /= 2;
    }
    // Measured on B200: a CTA streams one 32 KB step per 0.42 us at most (what its shared memory
    // holds in flight per memory round trip); the exchange through a cluster costs 2 us plus
    // 0.3 us per CTA of the cluster, through the scratch buffer 5.5 us (fences, an atomic and
    // the loads of the last CTA to arrive), both plus the partial tiles' own bytes.
    const double step_us = 0.42, hbm_bytes_per_us = 6.0e6;
    const double bytes = double(p.tiles) * kDecRows * double(k_bytes);
    const double hbm_us = bytes / hbm_bytes_per_us;
    const double whole_us = double((p.tiles + whole_ctas - 1) / whole_ctas) * p.ksteps * step_us;
    const auto split_us = [&](int parts, double exchange_us) {
        const double steps_us = double((p.ksteps + parts - 1) / parts) * step_us;
        return (hbm_us > steps_us ? hbm_us : steps_us) + exchange_us;
    };
    const double global_us = split_us(s, 5.5 + double(nact) / 64.0);
    const double cluster_us = sc > 1 ? split_us(sc, 2.0 + 0.3 * sc + double(nact) / 100.0) : 1e30;
    const double base_us = hbm_us > whole_us ? hbm_us : whole_us;
    const bool cluster = cluster_us <= global_us;
    if (force_split || (cluster ? cluster_us : global_us) < 0.85 * base_us) {
        const int parts = cluster ? sc : s;
        p.ctas = p.tiles * parts;
        p.aligned = 0;
        p.cluster = cluster ? parts : 0;
        p.fits32 = int64_t(p.tiles) * p.ksteps * p.ctas < (int64_t(1) << 32) ? 1 : 0;
    }
    return p;
}

// Host check of the unit deal, for tests: every unit is worked exactly once, the owner
// function agrees with the runs, and the scratch slots of one tile's contributors are distinct.
inline bool dec_plan_selfcheck(const DecPlan& p) {
    const int64_t units = int64_t(p.tiles) * p.ksteps;
    if (dec_begin(p, 0) != 0 || dec_begin(p, p.ctas) != units) return false;
    int64_t covered = 0;
    for (int c = 0; c < p.ctas; ++c) {
        DecWalk walk(p, c);
        DecSeg sg;
        int64_t u = dec_begin(p, c);
        int partial_slots[2] = {0, 0};
        while (walk.next(sg)) {
            if (int64_t(sg.tile) * p.ksteps + sg.k0 != u || sg.k1 <= sg.k0 || sg.k1 > p.ksteps) return false;
            for (int ks = sg.k0; ks < sg.k1; ++ks) {
                if (dec_owner(p, int64_t(sg.tile) * p.ksteps + ks) != c) return false;
            }
            if (sg.partial) {
                if (p.aligned) return false;
                const int slot = dec_slot(p, c, sg.tile);
                if (slot / 2 != c || ++partial_slots[slot & 1] > 1) return false;
                const int first = dec_owner(p, int64_t(sg.tile) * p.ksteps);
                const int last = dec_owner(p, int64_t(sg.tile + 1) * p.ksteps - 1);
                if (c < first || c > last || last == first) return false;
            }
            u += sg.k1 - sg.k0;
            covered += sg.k1 - sg.k0;
        }
        if (u != dec_begin(p, c + 1)) return false;
    }
    return covered == units;
}
