// Group-wise block-scale quantizer: bf16/fp16 [m, k] -> MXFP8 / MXFP4 / NVFP4
// codes plus UE8M0 / UE4M3 scales, emitted directly in the 128x4 SfAtom order
// the block-scaled tensor-core instructions consume.
//
// Same results, bit for bit, as the reference kernel
// (csrc/kernel/gemm/group_wise_quant.cu:123-231, csrc/common/mx_quant.cuh:104-150)
// as modelled by its own tests (tests/test_group_wise_quant.py:40-213), but a
// different decomposition: the reference gives one thread one whole group
// (lane-strided 16-byte loads); here a warp streams 2 KiB-contiguous row
// segments with fully coalesced 16-byte loads, 4 (or 2, or 1) lanes share a
// group and reduce its amax with warp shuffles, and the scale exponent is
// derived from the amax bit pattern with integer arithmetic instead of
// log2f/exp2f, so the result does not depend on fast-math code generation.
//
// HBM-bound: algorithmic bytes per element are 2 (read) + 1 + 1/32 (MXFP8),
// 2 + 1/2 + 1/32 (MXFP4), 2 + 1/2 + 1/16 (NVFP4).

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace hq {
namespace {

constexpr int kWarpsPerCta = 8;
constexpr int kThreads = kWarpsPerCta * 32;
constexpr int kColsPerWarp = 1024;  // elements of one row a warp handles
constexpr float kE4m3Max = 448.0f;
constexpr float kE2m1Max = 6.0f;
constexpr float kAmaxFloor = 1e-10f;  // reference: mx_quant.cuh:50

__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Pair-wise operations on a 32-bit word holding two T (x in the low half).
template <typename T>
struct Pair;

template <>
struct Pair<__nv_bfloat16> {
    static constexpr uint32_t kNegInf2 = 0xff80ff80u;
    static __device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b) {
        uint32_t r;
        asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));  // a NaN operand is ignored
        return r;
    }
    static constexpr uint32_t kInfBits = 0x7f80u;  // magnitudes from here on: infinity, NaN
    static __device__ __forceinline__ uint32_t abs2(uint32_t a) {
        uint32_t r;
        asm("abs.bf16x2 %0, %1;" : "=r"(r) : "r"(a));
        return r;
    }
    // max(a, |b|) and max(a, b) that return NaN when an operand is NaN
    static __device__ __forceinline__ uint32_t absmax2_nan(uint32_t a, uint32_t b) {
        uint32_t r;
        asm("{\n\t.reg .b32 t;\n\tabs.bf16x2 t, %2;\n\tmax.NaN.bf16x2 %0, %1, t;\n\t}" : "=r"(r) : "r"(a), "r"(b));
        return r;
    }
    static __device__ __forceinline__ uint32_t max2_nan(uint32_t a, uint32_t b) {
        uint32_t r;
        asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
        return r;
    }
    static __device__ __forceinline__ float lo(uint32_t w) { return __uint_as_float(w << 16); }
    static __device__ __forceinline__ float hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
};

template <>
struct Pair<__half> {
    static constexpr uint32_t kNegInf2 = 0xfc00fc00u;
    static __device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b) {
        uint32_t r;
        asm("max.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
        return r;
    }
    static constexpr uint32_t kInfBits = 0x7c00u;
    static __device__ __forceinline__ uint32_t abs2(uint32_t a) {
        uint32_t r;
        asm("abs.f16x2 %0, %1;" : "=r"(r) : "r"(a));
        return r;
    }
    static __device__ __forceinline__ uint32_t absmax2_nan(uint32_t a, uint32_t b) {
        uint32_t r;
        asm("{\n\t.reg .b32 t;\n\tabs.f16x2 t, %2;\n\tmax.NaN.f16x2 %0, %1, t;\n\t}" : "=r"(r) : "r"(a), "r"(b));
        return r;
    }
    static __device__ __forceinline__ uint32_t max2_nan(uint32_t a, uint32_t b) {
        uint32_t r;
        asm("max.NaN.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
        return r;
    }
    static __device__ __forceinline__ float lo(uint32_t w) {
        return __half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xffffu)));
    }
    static __device__ __forceinline__ float hi(uint32_t w) {
        return __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16)));
    }
};

// (a * s, b * s) as one packed instruction
__device__ __forceinline__ float2 mul2(float a, float b, float s) {
    float2 r;
    asm("{\n\t"
        ".reg .b64 t, u;\n\t"
        "mov.b64 t, {%2, %3};\n\t"
        "mov.b64 u, {%4, %4};\n\t"
        "mul.rn.f32x2 t, t, u;\n\t"
        "mov.b64 {%0, %1}, t;\n\t"
        "}"
        : "=f"(r.x), "=f"(r.y)
        : "f"(a), "f"(b), "f"(s));
    return r;
}
// (a * c, b * d) as one packed instruction
__device__ __forceinline__ float2 mul2v(float2 v, float2 w) {
    float2 r;
    asm("{\n\t"
        ".reg .b64 t, u;\n\t"
        "mov.b64 t, {%2, %3};\n\t"
        "mov.b64 u, {%4, %5};\n\t"
        "mul.rn.f32x2 t, t, u;\n\t"
        "mov.b64 {%0, %1}, t;\n\t"
        "}"
        : "=f"(r.x), "=f"(r.y)
        : "f"(v.x), "f"(v.y), "f"(w.x), "f"(w.y));
    return r;
}
// (a * a + c, b * b + d) as one packed instruction
__device__ __forceinline__ float2 fma2_sq(float2 v, float2 acc) {
    float2 r;
    asm("{\n\t"
        ".reg .b64 t, u;\n\t"
        "mov.b64 t, {%2, %3};\n\t"
        "mov.b64 u, {%4, %5};\n\t"
        "fma.rn.f32x2 u, t, t, u;\n\t"
        "mov.b64 {%0, %1}, u;\n\t"
        "}"
        : "=f"(r.x), "=f"(r.y)
        : "f"(v.x), "f"(v.y), "f"(acc.x), "f"(acc.y));
    return r;
}
// (a * s + 0, b * s + 0) as one packed instruction: the product, with the -0.0 that a zero
// factor gives turned into +0.0 (a product that underflows to zero keeps its sign: use it only
// where s is large enough for that not to happen, as the NVFP4 reciprocal scales are)
__device__ __forceinline__ float2 mul2_pos_zero(float a, float b, float s) {
    float2 r;
    asm("{\n\t"
        ".reg .b64 t, u, z;\n\t"
        "mov.b64 t, {%2, %3};\n\t"
        "mov.b64 u, {%4, %4};\n\t"
        "mov.b64 z, {%5, %5};\n\t"
        "fma.rn.f32x2 t, t, u, z;\n\t"
        "mov.b64 {%0, %1}, t;\n\t"
        "}"
        : "=f"(r.x), "=f"(r.y)
        : "f"(a), "f"(b), "f"(s), "f"(0.0f));
    return r;
}
// -0.0 -> +0.0, everything else unchanged.  (Written as two scalar adds: the
// packed add.rn.f32x2 with a zero operand does not survive ptxas.)
__device__ __forceinline__ float2 add_zero2(float2 v) {
    return make_float2(__fadd_rn(v.x, 0.0f), __fadd_rn(v.y, 0.0f));
}

// UE8M0 byte of ceil(log2(amax / D)) + 127 with the reference kernel's
// observed behaviour that an exact power of two below 1 comes out one higher
// (tests/test_group_wise_quant.py:40-53).  D = 1.75 * 2^8 (448) or 1.5 * 2^2
// (6): with B the biased exponent and M the mantissa field of amax,
//   amax / D = (1.M / 1.kk) * 2^(B - 127 - S)
// lies strictly inside a binade unless M equals D's mantissa, so
//   e = B - S - 1 + [M >= D.M] + 1, minus one when the quotient is an exact
// power of two that is >= 1.  Exact for every amax that comes from a bf16 or
// fp16 value and for the floor constant.
template <uint32_t kMant, int kShift>
__device__ __forceinline__ uint32_t ue8m0_of_amax(float amax) {
    const uint32_t u = __float_as_uint(amax);
    if (u >= 0x7f800000u) return 254u;  // an infinite amax saturates (fmaxf never returns NaN here)
    int e = int((u + (0x00800000u - kMant)) >> 23) - kShift;
    const bool exact_ge_one =
        (u & 0x007fffffu) == kMant && (u >> 23) >= uint32_t(127 + kShift);
    e -= exact_ge_one ? 1 : 0;
    return uint32_t(min(max(e, 0), 254));
}

// 2^(127 - e); e == 254 gives 0, which is what the reference's flush-to-zero
// exp2f(-127) returns.
__device__ __forceinline__ float inv_pow2(uint32_t e) {
    return __uint_as_float((254u - e) << 23);
}

__device__ __forceinline__ float clamp_sym(float x, float lim) {
    return fminf(fmaxf(x, -lim), lim);  // NaN -> -lim, as in the reference
}

// Two e2m1 codes (x in the low nibble), nearest with ties away from zero; a
// negative value that rounds to zero keeps its sign bit, -0.0 does not (the
// caller has added +0.0).  cvt rounds ties to even, so the midpoints that would
// go to the smaller (even) code - 0.25, 1.25, 2.5, 5 - are first moved one ulp
// outwards.
__device__ __forceinline__ uint32_t e2m1x2_half_away(float2 v) {
    const auto away = [](float x) {
        const uint32_t b = __float_as_uint(x);
        const uint32_t a = b & 0x7fffffffu;
        const bool tie = ((a - 0x3fa00000u) & 0xfe7fffffu) == 0u || a == 0x3e800000u;
        return __uint_as_float(b + (tie ? 1u : 0u));
    };
    return __nv_cvt_float2_to_fp4x2(make_float2(away(v.x), away(v.y)), __NV_E2M1, cudaRoundNearest);
}
// The same rounding for finite values, in three instructions: the lowest mantissa bit is set
// before the conversion.  Every midpoint between two e2m1 values is a float whose lowest bit is
// clear, so setting the bit moves a value that sits on a midpoint just past it, away from zero,
// and moves no other value onto or across a midpoint (the neighbour one ulp below a midpoint
// has the bit set already); round-to-nearest-even then gives round-half-away.  Zero becomes the
// smallest subnormal and still converts to zero.  Not for infinities (the bit would make a NaN):
// the caller's values are finite products of finite factors.
__device__ __forceinline__ uint32_t e2m1x2_half_away_finite(float2 v) {
    return __nv_cvt_float2_to_fp4x2(make_float2(__uint_as_float(__float_as_uint(v.x) | 1u),
                                                __uint_as_float(__float_as_uint(v.y) | 1u)),
                                    __NV_E2M1, cudaRoundNearest);
}
// Same for values that are exact products of a 16-bit float and a power of two
// and have already been scaled by 1 + 2^-23: such a value is never within an
// ulp below a midpoint, so plain round-to-nearest-even gives ties away.
__device__ __forceinline__ uint32_t e2m1x2_rne(float2 v) {
    return __nv_cvt_float2_to_fp4x2(v, __NV_E2M1, cudaRoundNearest);
}

__device__ __forceinline__ uint32_t e4m3x2(float x, float y) {
    return __nv_cvt_float2_to_fp8x2(make_float2(x, y), __NV_SATFINITE, __NV_E4M3);
}

// quantize_piece for a group that holds a NaN or an infinity (rare).  The
// lanes that share the group call it together; other lanes of the warp may be elsewhere, so
// the shuffles name only the group's lanes.
template <typename T, int kMode>
__device__ __forceinline__ uint32_t quantize_piece_special(
    const uint32_t (&w)[(kMode == HQ_MODE_W4A4_NVFP4 ? 16 : 8) / 2],
    uint32_t (&codes)[(kMode == HQ_MODE_W4A4_NVFP4 ? 16 : 8) / 2]) {
    constexpr bool kNv = kMode == HQ_MODE_W4A4_NVFP4;
    constexpr bool kFp4 = kMode != HQ_MODE_W8A8_MXFP8;
    constexpr int kWords = (kNv ? 16 : 8) / 2;
    using P = Pair<T>;
    const uint32_t group_lanes = kNv ? 0u : 0xfu << (threadIdx.x & 28u);
    // group amax on the packed 16-bit values (NaN operands are ignored, as fmaxf does)
    uint32_t mx = w[0] & 0x7fff7fffu;
#pragma unroll
    for (int i = 1; i < kWords; ++i) mx = P::max2(mx, w[i] & 0x7fff7fffu);
    mx = P::max2(mx, __byte_perm(mx, 0, 0x1032));
    if constexpr (!kNv) {
        mx = P::max2(mx, __shfl_xor_sync(group_lanes, mx, 1));
        mx = P::max2(mx, __shfl_xor_sync(group_lanes, mx, 2));
    }
    const float amax = fmaxf(P::lo(mx), kAmaxFloor);

    uint32_t sf_byte;
    float inv;
    if constexpr (kMode == HQ_MODE_W8A8_MXFP8) {
        sf_byte = ue8m0_of_amax<0x00600000u, 8>(amax);
        inv = inv_pow2(sf_byte);
    } else if constexpr (kMode == HQ_MODE_W4A4_MXFP4) {
        sf_byte = ue8m0_of_amax<0x00400000u, 2>(amax);
        inv = inv_pow2(sf_byte);
    } else {
        // amax / 6, correctly rounded: a product with 1/6 and one Newton correction of the quotient
        // (checked against the division for every bf16 and fp16 amax and for the floor)
        constexpr float kSixth = 1.0f / 6.0f;
        const float q0 = __fmul_rn(amax, kSixth);
        const float quot = __fmaf_rn(__fmaf_rn(-kE2m1Max, q0, amax), kSixth, q0);
        const float s = fminf(quot, kE4m3Max);
        sf_byte = __nv_cvt_float_to_fp8(s, __NV_SATFINITE, __NV_E4M3);
        // UE4M3 may round a tiny scale to 0: smallest positive code (2^-9)
        if (sf_byte == 0u) sf_byte = 1u;
        const float dec = __half2float(__half(__nv_cvt_fp8_to_halfraw(
            static_cast<__nv_fp8_storage_t>(sf_byte), __NV_E4M3)));
        inv = __frcp_rn(dec);
    }

    // The reference clamps every scaled value with fminf(fmaxf(x, -MAX), MAX), which
    // also turns NaN into -MAX.  Finite values never exceed MAX after scaling (or
    // saturate in the conversion), so only the NaN rule needs work: NaN is replaced
    // by -inf in the packed input, which scales to -inf and saturates to -MAX.  A
    // group that holds an infinity has inv == 0 (inf * 0 = NaN) and takes the
    // literal clamp.
    if (inv != 0.0f) {
        const float mult = kMode == HQ_MODE_W4A4_MXFP4 ? inv * (1.0f + 1.1920929e-7f) : inv;
#pragma unroll
        for (int i = 0; i < kWords; ++i) {
            const uint32_t g = P::max2(w[i], P::kNegInf2);
            const float2 x = mul2(P::lo(g), P::hi(g), mult);
            if constexpr (kMode == HQ_MODE_W8A8_MXFP8) {
                codes[i] = e4m3x2(x.x, x.y);
            } else if constexpr (kMode == HQ_MODE_W4A4_MXFP4) {
                codes[i] = e2m1x2_rne(add_zero2(x));
            } else {
                codes[i] = e2m1x2_half_away(add_zero2(x));
            }
        }
    } else {
        const float lim = kFp4 ? kE2m1Max : kE4m3Max;
#pragma unroll
        for (int i = 0; i < kWords; ++i) {
            const float a = clamp_sym(__fmul_rn(P::lo(w[i]), inv), lim);
            const float b = clamp_sym(__fmul_rn(P::hi(w[i]), inv), lim);
            if constexpr (!kFp4) {
                codes[i] = e4m3x2(a, b);
            } else {
                codes[i] = e2m1x2_half_away(add_zero2(make_float2(a, b)));
            }
        }
    }

    return sf_byte;
}

// Scale byte and codes of the kEpl = 2 * kWords values one lane holds of a
// quantisation group (packed two per word): 4 lanes share a 32-element group
// and reduce its amax with two shuffles, NVFP4 gives a lane a whole 16-element
// group.  codes[i] holds the two codes of word i: 16 bits (e4m3) or 8 bits
// (e2m1).  Every lane of the warp must call it.
//
// The maximum of the magnitudes is taken with the NaN-propagating max, so one compare of
// the result tells whether the group holds a NaN or an infinity.  Such groups go to
// quantize_piece_special, which implements the reference's clamp (NaN -> -MAX, infinities
// saturate) literally; every other group holds finite values only, whose scaled values
// cannot overflow: no clamp, no NaN rule, and the reciprocal scale is never zero.
template <typename T, int kMode>
__device__ __forceinline__ uint32_t quantize_piece(
    const uint32_t (&w)[(kMode == HQ_MODE_W4A4_NVFP4 ? 16 : 8) / 2],
    uint32_t (&codes)[(kMode == HQ_MODE_W4A4_NVFP4 ? 16 : 8) / 2]) {
    constexpr bool kNv = kMode == HQ_MODE_W4A4_NVFP4;
    constexpr int kWords = (kNv ? 16 : 8) / 2;
    using P = Pair<T>;
    uint32_t mx = P::abs2(w[0]);
#pragma unroll
    for (int i = 1; i < kWords; ++i) mx = P::absmax2_nan(mx, w[i]);
    mx = P::max2_nan(mx, __byte_perm(mx, 0, 0x1032));
    if constexpr (!kNv) {
        mx = P::max2_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = P::max2_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    }
    if ((mx & 0x7fffu) >= P::kInfBits) return quantize_piece_special<T, kMode>(w, codes);
    const float amax = fmaxf(P::lo(mx), kAmaxFloor);

    uint32_t sf_byte;
    float inv;
    if constexpr (kMode == HQ_MODE_W8A8_MXFP8) {
        sf_byte = ue8m0_of_amax<0x00600000u, 8>(amax);
        inv = inv_pow2(sf_byte);
    } else if constexpr (kMode == HQ_MODE_W4A4_MXFP4) {
        sf_byte = ue8m0_of_amax<0x00400000u, 2>(amax);
        // (1 + 2^-23: see e2m1x2_rne)
        inv = inv_pow2(sf_byte) * (1.0f + 1.1920929e-7f);
    } else {
        // amax / 6, correctly rounded: a product with 1/6 and one Newton correction of the quotient
        // (checked against the division for every bf16 and fp16 amax and for the floor)
        constexpr float kSixth = 1.0f / 6.0f;
        const float q0 = __fmul_rn(amax, kSixth);
        const float quot = __fmaf_rn(__fmaf_rn(-kE2m1Max, q0, amax), kSixth, q0);
        sf_byte = __nv_cvt_float_to_fp8(fminf(quot, kE4m3Max), __NV_SATFINITE, __NV_E4M3);
        // UE4M3 may round a tiny scale to 0: smallest positive code (2^-9)
        if (sf_byte == 0u) sf_byte = 1u;
        const float dec = __half2float(__half(__nv_cvt_fp8_to_halfraw(
            static_cast<__nv_fp8_storage_t>(sf_byte), __NV_E4M3)));
        inv = __frcp_rn(dec);
    }

#pragma unroll
    for (int i = 0; i < kWords; ++i) {
        if constexpr (kMode == HQ_MODE_W8A8_MXFP8) {
            const float2 x = mul2(P::lo(w[i]), P::hi(w[i]), inv);
            codes[i] = e4m3x2(x.x, x.y);
        } else if constexpr (kMode == HQ_MODE_W4A4_MXFP4) {
            // (a product that underflows to -0.0 must come out as +0.0 too: multiply, then add zero)
            codes[i] = e2m1x2_rne(add_zero2(mul2(P::lo(w[i]), P::hi(w[i]), inv)));
        } else {
            codes[i] = e2m1x2_half_away_finite(mul2_pos_zero(P::lo(w[i]), P::hi(w[i]), inv));
        }
    }
    return sf_byte;
}

// One warp quantizes kColsPerWarp consecutive elements of one row.  A lane
// handles kEpl elements per piece: 8 for the 32-element groups (4 lanes per
// group), 16 for NVFP4 (one lane per group).  Every address is a per-lane base
// computed once plus a compile-time offset per piece.  kFull: the whole
// segment lies inside the row, no column predicates.
template <typename T, int kMode, bool kSwizzle, bool kFull>
__device__ __forceinline__ void quantize_segment(const T* __restrict__ in_row,
                                                 uint8_t* __restrict__ q_row,
                                                 uint8_t* __restrict__ sf_lane, int col0, int k,
                                                 int lane) {
    constexpr bool kNv = kMode == HQ_MODE_W4A4_NVFP4;
    constexpr bool kFp4 = kMode != HQ_MODE_W8A8_MXFP8;
    constexpr int kEpl = kNv ? 16 : 8;
    constexpr int kPieces = kColsPerWarp / (32 * kEpl);  // 4 or 2
    constexpr int kGroup = kNv ? 16 : 32;
    constexpr int kWords = kEpl / 2;
    using P = Pair<T>;

    const uint4* const src = reinterpret_cast<const uint4*>(in_row + col0 + lane * kEpl);
    const int lane_col = col0 + lane * kEpl;
    uint4 raw[kPieces][kEpl / 8];
#pragma unroll
    for (int p = 0; p < kPieces; ++p) {
#pragma unroll
        for (int h = 0; h < kEpl / 8; ++h) {
            const bool active = kFull || lane_col + p * 32 * kEpl < k;
            raw[p][h] = active ? ld_stream(src + p * 4 * kEpl + h) : make_uint4(0, 0, 0, 0);
        }
    }

#pragma unroll
    for (int p = 0; p < kPieces; ++p) {
        const bool active = kFull || lane_col + p * 32 * kEpl < k;
        uint32_t w[kWords];
#pragma unroll
        for (int h = 0; h < kEpl / 8; ++h) {
            w[4 * h + 0] = raw[p][h].x;
            w[4 * h + 1] = raw[p][h].y;
            w[4 * h + 2] = raw[p][h].z;
            w[4 * h + 3] = raw[p][h].w;
        }
        uint32_t codes[kWords];
        const uint32_t sf_byte = quantize_piece<T, kMode>(w, codes);

        if constexpr (!kFp4) {
            // 4 x (2 codes in 16 bits) -> 2 words; 8 bytes per lane and piece
            const uint32_t q0 = __byte_perm(codes[0], codes[1], 0x5410);
            const uint32_t q1 = __byte_perm(codes[2], codes[3], 0x5410);
            if (active) {
                reinterpret_cast<uint2*>(q_row + col0 + lane * 8)[p * 32] = make_uint2(q0, q1);
            }
        } else {
            // one byte per pair -> one word per 8 elements
            uint32_t q[kWords / 4];
#pragma unroll
            for (int h = 0; h < kWords / 4; ++h) {
                // byte 0 of four code words -> one word
                q[h] = __byte_perm(__byte_perm(codes[4 * h], codes[4 * h + 1], 0x0040),
                                   __byte_perm(codes[4 * h + 2], codes[4 * h + 3], 0x0040), 0x5410);
            }
            if (active) {
                uint8_t* const dst = q_row + (col0 >> 1) + lane * (kEpl / 2);
                if constexpr (kNv) {
                    reinterpret_cast<uint2*>(dst)[p * 32] = make_uint2(q[0], q[kWords / 4 - 1]);
                } else {
                    reinterpret_cast<uint32_t*>(dst)[p * 32] = q[0];
                }
            }
        }

        if constexpr (kSwizzle) {
            // the four scale bytes of one SfAtom word sit in lanes L, L+s, L+2s, L+3s;
            // consecutive words of a row are 512 bytes apart
            constexpr int s = kNv ? 1 : 4;
            uint32_t word = sf_byte;
            word |= __shfl_down_sync(0xffffffffu, word, s) << 8;
            word |= __shfl_down_sync(0xffffffffu, word, 2 * s) << 16;
            if (active && (lane & (4 * s - 1)) == 0) {
                *reinterpret_cast<uint32_t*>(sf_lane + p * (8 * kEpl / kGroup) * 512) = word;
            }
        } else {
            const bool lead = kNv ? true : (lane & 3) == 0;
            if (active && lead) sf_lane[p * (32 * kEpl / kGroup)] = uint8_t(sf_byte);
        }
    }
}

template <typename T, int kMode, bool kSwizzle>
__global__ void __launch_bounds__(kThreads)
group_wise_quant_kernel(const T* __restrict__ input, int64_t ld,
                        uint8_t* __restrict__ out_q, uint8_t* __restrict__ out_sf,
                        int64_t m, int64_t rows_total, int k, int kb_dim) {
    constexpr bool kNv = kMode == HQ_MODE_W4A4_NVFP4;
    constexpr bool kFp4 = kMode != HQ_MODE_W8A8_MXFP8;
    constexpr int kEpl = kNv ? 16 : 8;
    constexpr int kPieces = kColsPerWarp / (32 * kEpl);
    constexpr int kGroup = kNv ? 16 : 32;

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t row = int64_t(blockIdx.x) * kWarpsPerCta + warp;
    const int col0 = blockIdx.y * kColsPerWarp;

    // per-lane base of this lane's scale bytes for piece 0
    uint8_t* sf_lane;
    if constexpr (kSwizzle) {
        sf_lane = out_sf + ((row >> 7) * (kb_dim >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 +
                  int64_t((col0 + lane * kEpl) / (4 * kGroup)) * 512;
    } else {
        sf_lane = out_sf + row * int64_t(kb_dim) + (col0 + lane * kEpl) / kGroup;
    }

    // The first global access is below: with a programmatic launch the index
    // math above overlaps the tail of the producing kernel.  The kernel behind this one may
    // start its own set-up at once (it still waits for this whole grid before it reads
    // anything): a decode GEMM then has its prologue, and with early weight loads its first
    // stages, behind it when the few CTAs of an activation's quantizer are done.
    pdl_launch_dependents();
    pdl_wait();

    if (row >= rows_total) return;

    if (row >= m) {
        // padding rows of the last SfAtom (swizzled layout only): zero scales
        if constexpr (kSwizzle) {
            const bool lead = kNv ? (lane & 3) == 0 : (lane & 15) == 0;
#pragma unroll
            for (int p = 0; p < kPieces; ++p) {
                if (lead && col0 + (p * 32 + lane) * kEpl < k) {
                    *reinterpret_cast<uint32_t*>(sf_lane + p * (8 * kEpl / kGroup) * 512) = 0u;
                }
            }
        }
        return;
    }

    const T* const in_row = input + row * ld;
    uint8_t* const q_row = out_q + row * int64_t(kFp4 ? (k >> 1) : k);
    if (col0 + kColsPerWarp <= k) {
        quantize_segment<T, kMode, kSwizzle, true>(in_row, q_row, sf_lane, col0, k, lane);
    } else {
        quantize_segment<T, kMode, kSwizzle, false>(in_row, q_row, sf_lane, col0, k, lane);
    }
}

// RMSNorm fused with the MXFP8 quantizer: y = bf16(x * rsqrt(mean(x^2) + eps) * gamma)
// quantised exactly as group_wise_quant(y) would, reading x once.  Replaces the
// reference's rms_norm_quant_kernel (csrc/kernel/gemm/rms_norm_quant.cu:44-107):
// there one thread owns a whole 32-element group; here one CTA owns a row, a lane
// 8 consecutive elements (coalesced 16-byte loads, the row stays in registers),
// the sum of squares is reduced by shuffles and one shared-memory pass, and the
// quantisation is the quantizer's own per-piece code.
constexpr int kRmsMaxK = 8192;

// kPieces 8-element pieces per thread: piece p of thread t covers columns
// (p * blockDim.x + t) * 8 .. + 8, so every load instruction of a warp is one
// contiguous 512-byte run and several rows are in flight per SM.
template <bool kSwizzle, int kPieces>
__global__ void __launch_bounds__(kRmsMaxK / 8 / kPieces)
rms_norm_quant_kernel(const __nv_bfloat16* __restrict__ x, int64_t ld,
                      const __nv_bfloat16* __restrict__ gamma, float eps, int64_t m, int k,
                      uint8_t* __restrict__ q, uint8_t* __restrict__ sf) {
    __shared__ float warp_sums[kRmsMaxK / 8 / 32];
    const int64_t row = blockIdx.x;
    const int t = threadIdx.x;
    const int lane = t & 31;
    const int threads = blockDim.x;
    const int kb_dim = k >> 5;
    using P = Pair<__nv_bfloat16>;

    uint8_t* sf_row;
    if constexpr (kSwizzle) {
        sf_row = sf + ((row >> 7) * (kb_dim >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4;
    } else {
        sf_row = sf + row * int64_t(kb_dim);
    }
    // gamma does not depend on the producing kernel
    uint4 gw[kPieces];
#pragma unroll
    for (int p = 0; p < kPieces; ++p) {
        const int col = (p * threads + t) * 8;
        gw[p] = col < k ? __ldg(reinterpret_cast<const uint4*>(gamma + col)) : make_uint4(0, 0, 0, 0);
    }

    pdl_launch_dependents();
    pdl_wait();

    if (row >= m) {  // padding rows of the last SfAtom (swizzled layout only)
        if constexpr (kSwizzle) {
#pragma unroll
            for (int p = 0; p < kPieces; ++p) {
                const int col = (p * threads + t) * 8;
                if (col < k && (lane & 15) == 0) *reinterpret_cast<uint32_t*>(sf_row + int64_t(col >> 7) * 512) = 0u;
            }
        }
        return;
    }

    uint4 raw[kPieces];
#pragma unroll
    for (int p = 0; p < kPieces; ++p) {
        const int col = (p * threads + t) * 8;
        raw[p] = col < k ? ld_stream(x + row * ld + col) : make_uint4(0, 0, 0, 0);
    }
    // the row as floats (kept for the second pass) and its sum of squares, two lanes of a
    // packed accumulator that are added at the end
    float2 xf[kPieces][4];
    float2 acc2 = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int p = 0; p < kPieces; ++p) {
        const uint32_t xw[4] = {raw[p].x, raw[p].y, raw[p].z, raw[p].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            xf[p][i] = make_float2(P::lo(xw[i]), P::hi(xw[i]));
            acc2 = fma2_sq(xf[p][i], acc2);
        }
    }
    float sum_sq = acc2.x + acc2.y;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) sum_sq += __shfl_xor_sync(0xffffffffu, sum_sq, s);
    const int warps = threads >> 5;
    if (warps > 1) {
        if (lane == 0) warp_sums[t >> 5] = sum_sq;
        __syncthreads();
        sum_sq = 0.0f;
        for (int i = 0; i < warps; ++i) sum_sq += warp_sums[i];
    }
    const float rrms = rsqrtf(sum_sq / float(k) + eps);
    const float2 rrms2 = make_float2(rrms, rrms);

#pragma unroll
    for (int p = 0; p < kPieces; ++p) {
        const int col = (p * threads + t) * 8;
        const bool active = col < k;
        const uint32_t gws[4] = {gw[p].x, gw[p].y, gw[p].z, gw[p].w};
        uint32_t yw[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            // (x * rrms) * gamma, each product rounded to float32, as two packed multiplies
            const float2 y2 = mul2v(mul2v(xf[p][i], rrms2), make_float2(P::lo(gws[i]), P::hi(gws[i])));
            const __nv_bfloat162 y = __float22bfloat162_rn(y2);
            yw[i] = *reinterpret_cast<const uint32_t*>(&y);
        }
        uint32_t codes[4];
        const uint32_t sf_byte = quantize_piece<__nv_bfloat16, HQ_MODE_W8A8_MXFP8>(yw, codes);
        if (active) {
            *reinterpret_cast<uint2*>(q + row * int64_t(k) + col) =
                make_uint2(__byte_perm(codes[0], codes[1], 0x5410), __byte_perm(codes[2], codes[3], 0x5410));
        }
        if constexpr (kSwizzle) {
            uint32_t word = sf_byte;
            word |= __shfl_down_sync(0xffffffffu, word, 4) << 8;
            word |= __shfl_down_sync(0xffffffffu, word, 8) << 16;
            if (active && (lane & 15) == 0) *reinterpret_cast<uint32_t*>(sf_row + int64_t(col >> 7) * 512) = word;
        } else {
            if (active && (lane & 3) == 0) sf_row[col >> 5] = uint8_t(sf_byte);
        }
    }
}

template <typename T, int kMode>
cudaError_t launch_mode(const T* in, int64_t ld, uint8_t* q, uint8_t* sf, int64_t m,
                        int k, bool swizzle, bool pdl, cudaStream_t stream) {
    const int kb_dim = k / (kMode == HQ_MODE_W4A4_NVFP4 ? 16 : 32);
    const int64_t rows_total = swizzle ? hq_sf_rows(m) : m;
    const dim3 grid(unsigned((rows_total + kWarpsPerCta - 1) / kWarpsPerCta),
                    unsigned((k + kColsPerWarp - 1) / kColsPerWarp));
    if (swizzle) {
        return launch(group_wise_quant_kernel<T, kMode, true>, grid, dim3(kThreads), 0,
                      stream, pdl, 1, in, ld, q, sf, m, rows_total, k, kb_dim);
    }
    return launch(group_wise_quant_kernel<T, kMode, false>, grid, dim3(kThreads), 0,
                  stream, pdl, 1, in, ld, q, sf, m, rows_total, k, kb_dim);
}

template <typename T>
cudaError_t launch_dtype(const void* in, int64_t ld, void* q, void* sf, int64_t m, int k,
                         int mode, bool swizzle, bool pdl, cudaStream_t stream) {
    const T* p = static_cast<const T*>(in);
    uint8_t* pq = static_cast<uint8_t*>(q);
    uint8_t* psf = static_cast<uint8_t*>(sf);
    switch (mode) {
        case HQ_MODE_W8A8_MXFP8:
            return launch_mode<T, HQ_MODE_W8A8_MXFP8>(p, ld, pq, psf, m, k, swizzle, pdl, stream);
        case HQ_MODE_W4A4_MXFP4:
            return launch_mode<T, HQ_MODE_W4A4_MXFP4>(p, ld, pq, psf, m, k, swizzle, pdl, stream);
        default:
            return launch_mode<T, HQ_MODE_W4A4_NVFP4>(p, ld, pq, psf, m, k, swizzle, pdl, stream);
    }
}

}  // namespace
}  // namespace hq

extern "C" int hq_parse_mode(const char* mode) {
    if (mode == nullptr) return -1;
    if (strcmp(mode, "w8a8-mxfp8") == 0) return HQ_MODE_W8A8_MXFP8;
    if (strcmp(mode, "w4a4-mxfp4") == 0) return HQ_MODE_W4A4_MXFP4;
    if (strcmp(mode, "w4a4-nvfp4") == 0) return HQ_MODE_W4A4_NVFP4;
    return -1;
}

extern "C" int hq_group_size(int mode) {
    switch (mode) {
        case HQ_MODE_W8A8_MXFP8:
        case HQ_MODE_W4A4_MXFP4:
            return 32;
        case HQ_MODE_W4A4_NVFP4:
            return 16;
        default:
            return 0;
    }
}

extern "C" int64_t hq_sf_rows(int64_t m) { return (m + 127) / 128 * 128; }

extern "C" int hq_group_wise_quant(const void* input, int64_t ld_elems, int in_dtype,
                                   int64_t m, int64_t k, int mode, int use_swizzle,
                                   int use_pdl, void* out_q, void* out_sf, int device,
                                   void* stream, char* err, size_t errlen) {
    using hq::fail;
    const int group = hq_group_size(mode);
    if (group == 0) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "Unsupported quantization mode: %d. Expected 'w8a8-mxfp8', "
                    "'w4a4-mxfp4' or 'w4a4-nvfp4'.", mode);
    }
    if (in_dtype != HQ_DTYPE_BF16 && in_dtype != HQ_DTYPE_FP16) {
        return fail(err, errlen, HQ_ERR_INVALID, "input dtype must be bfloat16 or float16");
    }
    if (m < 0 || k < 0 || k > INT32_MAX) {
        return fail(err, errlen, HQ_ERR_INVALID, "input must be a 2D tensor of shape [m, k]");
    }
    if (k % group != 0) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "k must be divisible by the quantization group size (%d), got k=%lld",
                    group, static_cast<long long>(k));
    }
    const int64_t kb_dim = k / group;
    if (use_swizzle && kb_dim % 4 != 0) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "scale kb_dim must be divisible by 4 for CUTLASS SfAtom layout, got %lld",
                    static_cast<long long>(kb_dim));
    }
    if (m == 0 || k == 0) return HQ_OK;
    if (input == nullptr || out_q == nullptr || out_sf == nullptr) {
        return fail(err, errlen, HQ_ERR_INVALID, "null pointer argument");
    }
    if (ld_elems < k || (ld_elems * 2) % 16 != 0 || !hq::aligned(input, 16)) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "input rows must be contiguous and 16-byte aligned");
    }
    if (!hq::aligned(out_q, 16) || !hq::aligned(out_sf, use_swizzle ? 16 : 1)) {
        return fail(err, errlen, HQ_ERR_INVALID,
                    "output_quant / output_sf must be 16-byte aligned");
    }
    if ((m + 7) / 8 > INT32_MAX) {
        return fail(err, errlen, HQ_ERR_INVALID, "m is too large for one launch");
    }
    const hq::DeviceGuard guard(device);
    if (!guard.ok()) return fail(err, errlen, HQ_ERR_CUDA, "cannot select CUDA device %d", device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const cudaError_t e =
        in_dtype == HQ_DTYPE_BF16
            ? hq::launch_dtype<__nv_bfloat16>(input, ld_elems, out_q, out_sf, m, int(k), mode,
                                              use_swizzle != 0, use_pdl != 0, s)
            : hq::launch_dtype<__half>(input, ld_elems, out_q, out_sf, m, int(k), mode,
                                       use_swizzle != 0, use_pdl != 0, s);
    HQ_CUDA_TRY(e);
    return HQ_OK;
}

extern "C" int hq_rms_norm_quant(const void* input, int64_t ld_elems, const void* weight, float eps,
                                 int64_t m, int64_t k, int use_swizzle, int use_pdl, void* out_q,
                                 void* out_sf, int device, void* stream, char* err, size_t errlen) {
    using hq::fail;
    if (m < 0 || k <= 0) {
        return fail(err, errlen, HQ_ERR_INVALID, "input must be a 2D bfloat16 tensor [M, K]");
    }
    if (k % 128 != 0 || k > hq::kRmsMaxK) {
        return fail(err, errlen, HQ_ERR_INVALID, "K must be a multiple of 128 and at most %d, got %lld",
                    hq::kRmsMaxK, static_cast<long long>(k));
    }
    const int64_t rows_total = use_swizzle ? hq_sf_rows(m) : m;
    if (rows_total == 0) return HQ_OK;
    if (input == nullptr || weight == nullptr || out_q == nullptr || out_sf == nullptr) {
        return fail(err, errlen, HQ_ERR_INVALID, "null pointer argument");
    }
    if (ld_elems < k || (ld_elems * 2) % 16 != 0 || !hq::aligned(input, 16)) {
        return fail(err, errlen, HQ_ERR_INVALID, "input rows must be contiguous and 16-byte aligned");
    }
    if (!hq::aligned(weight, 16) || !hq::aligned(out_q, 16) || !hq::aligned(out_sf, use_swizzle ? 16 : 1)) {
        return fail(err, errlen, HQ_ERR_INVALID, "weight, q and sf must be 16-byte aligned");
    }
    if (rows_total > INT32_MAX) return fail(err, errlen, HQ_ERR_INVALID, "m is too large for one launch");
    const hq::DeviceGuard guard(device);
    if (!guard.ok()) return fail(err, errlen, HQ_ERR_CUDA, "cannot select CUDA device %d", device);
    // 1, 2 or 4 pieces of 8 elements per thread, at least 128 threads per row when K allows
    const int pieces = k >= 4096 ? 4 : (k >= 2048 ? 2 : 1);
    const int threads = int((k / (8 * pieces) + 31) / 32 * 32);
    const auto* x = static_cast<const __nv_bfloat16*>(input);
    const auto* g = static_cast<const __nv_bfloat16*>(weight);
    auto* q = static_cast<uint8_t*>(out_q);
    auto* sf = static_cast<uint8_t*>(out_sf);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const dim3 grid(static_cast<unsigned>(rows_total));
    cudaError_t e;
#define HQ_RMS_LAUNCH(SW, PC)                                                                          \
    e = hq::launch(hq::rms_norm_quant_kernel<SW, PC>, grid, dim3(threads), 0, s, use_pdl != 0, 1, x, \
                   ld_elems, g, eps, m, int(k), q, sf)
    if (use_swizzle) {
        if (pieces == 4) HQ_RMS_LAUNCH(true, 4);
        else if (pieces == 2) HQ_RMS_LAUNCH(true, 2);
        else HQ_RMS_LAUNCH(true, 1);
    } else {
        if (pieces == 4) HQ_RMS_LAUNCH(false, 4);
        else if (pieces == 2) HQ_RMS_LAUNCH(false, 2);
        else HQ_RMS_LAUNCH(false, 1);
    }
#undef HQ_RMS_LAUNCH
    HQ_CUDA_TRY(e);
    return HQ_OK;
}
