// Device-side helpers shared by the TOSA kernels: typed element access with the tensor
// layer's out-of-range rules and the RESCALE arithmetic.
//
// Access rules follow tensor/shaders/tensor.glsl:24-86 of the reference: coordinates are
// unsigned; a read with any coordinate >= shape yields 0; a write out of range is dropped.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "../ops.hpp"

namespace mlel {

constexpr int kNumSMs = 148; // B200
constexpr int kThreads = 256;

inline int gridFor(int64_t work, int perBlock = kThreads, int maxBlocksPerSM = 8) {
    int64_t blocks = (work + perBlock - 1) / perBlock;
    const int64_t cap = int64_t(kNumSMs) * maxBlocksPerSM;
    if (blocks > cap) {
        blocks = cap;
    }
    return blocks < 1 ? 1 : int(blocks);
}

__host__ __device__ inline int dtypeSize(int32_t dtype) {
    switch (dtype) {
    case MLEL_BOOL:
    case MLEL_I8:
    case MLEL_U8:
        return 1;
    case MLEL_I16:
    case MLEL_U16:
    case MLEL_F16:
    case MLEL_BF16:
        return 2;
    case MLEL_I32:
    case MLEL_U32:
    case MLEL_F32:
        return 4;
    case MLEL_I64:
        return 8;
    default:
        return 0;
    }
}

// Row-major unravel of a linear element offset (last dimension fastest).
__device__ inline void unravel(const TView &t, uint32_t off, uint32_t *idx) {
#pragma unroll
    for (int i = kMaxRank - 1; i >= 0; --i) {
        if (i < t.rank) {
            idx[i] = off % t.dims[i];
            off /= t.dims[i];
        }
    }
}

// Byte offset of a coordinate, or -1 when any coordinate is out of range.
__device__ inline int64_t offsetOf(const TView &t, const uint32_t *c) {
    int64_t off = 0;
#pragma unroll
    for (int i = 0; i < kMaxRank; ++i) {
        if (i < t.rank) {
            if (c[i] >= t.dims[i]) {
                return -1;
            }
            off += int64_t(c[i]) * t.strides[i];
        }
    }
    return off;
}

__device__ inline int64_t loadIntAt(const TView &t, int64_t off) {
    const char *p = t.ptr + off;
    switch (t.dtype) {
    case MLEL_BOOL:
    case MLEL_I8:
        return *reinterpret_cast<const int8_t *>(p);
    case MLEL_U8:
        return *reinterpret_cast<const uint8_t *>(p);
    case MLEL_I16:
        return *reinterpret_cast<const int16_t *>(p);
    case MLEL_U16:
    case MLEL_F16:
    case MLEL_BF16:
        return *reinterpret_cast<const uint16_t *>(p);
    case MLEL_I32:
        return *reinterpret_cast<const int32_t *>(p);
    case MLEL_U32:
    case MLEL_F32:
        return *reinterpret_cast<const uint32_t *>(p);
    default:
        return *reinterpret_cast<const int64_t *>(p);
    }
}

__device__ inline int64_t loadInt(const TView &t, const uint32_t *c) {
    const int64_t off = offsetOf(t, c);
    return off < 0 ? 0 : loadIntAt(t, off);
}

// Narrowing store with the constructor of the tensor's own type (wraps).
__device__ inline void storeIntAt(const TView &t, int64_t off, int64_t v) {
    char *p = t.ptr + off;
    switch (dtypeSize(t.dtype)) {
    case 1:
        *reinterpret_cast<int8_t *>(p) = int8_t(uint8_t(uint64_t(v)));
        break;
    case 2:
        *reinterpret_cast<int16_t *>(p) = int16_t(uint16_t(uint64_t(v)));
        break;
    case 4:
        *reinterpret_cast<int32_t *>(p) = int32_t(uint32_t(uint64_t(v)));
        break;
    default:
        *reinterpret_cast<int64_t *>(p) = v;
        break;
    }
}

__device__ inline void storeInt(const TView &t, const uint32_t *c, int64_t v) {
    const int64_t off = offsetOf(t, c);
    if (off >= 0) {
        storeIntAt(t, off, v);
    }
}

__host__ __device__ inline int64_t wrapTo(int32_t dtype, int64_t v) {
    switch (dtype) {
    case MLEL_BOOL:
        return v != 0 ? 1 : 0;
    case MLEL_I8:
        return int8_t(uint8_t(uint64_t(v)));
    case MLEL_U8:
        return uint8_t(uint64_t(v));
    case MLEL_I16:
        return int16_t(uint16_t(uint64_t(v)));
    case MLEL_U16:
        return uint16_t(uint64_t(v));
    case MLEL_I32:
        return int32_t(uint32_t(uint64_t(v)));
    case MLEL_U32:
        return uint32_t(uint64_t(v));
    default:
        return v;
    }
}

__host__ __device__ inline int64_t typeLowest(int32_t dtype) {
    switch (dtype) {
    case MLEL_I8:
        return -128;
    case MLEL_I16:
        return -32768;
    case MLEL_I32:
        return -2147483647ll - 1;
    case MLEL_I64:
        return int64_t(0x8000000000000000ull);
    default:
        return 0;
    }
}

__host__ __device__ inline int64_t typeMax(int32_t dtype) {
    switch (dtype) {
    case MLEL_BOOL:
        return 1;
    case MLEL_I8:
        return 127;
    case MLEL_U8:
        return 255;
    case MLEL_I16:
        return 32767;
    case MLEL_U16:
        return 65535;
    case MLEL_I32:
        return 2147483647ll;
    case MLEL_U32:
        return 4294967295ll;
    default:
        return int64_t(0x7fffffffffffffffull);
    }
}

// TOSA RESCALE scaling step as the reference computes it (rescale.comp:27-46): 64-bit
// product, rounding term 1 << (shift-1) (0 for shift 0), +-(1<<30) when double rounding
// and shift > 31, arithmetic shift, truncation to 32 bits.
__host__ __device__ inline int32_t applyScale(int64_t value, int32_t multiplier, int32_t shift, bool doubleRound) {
    int64_t round = shift > 0 ? int64_t(1ull << ((shift - 1) & 63)) : 0;
    if (doubleRound && shift > 31) {
        round += value >= 0 ? (int64_t(1) << 30) : -(int64_t(1) << 30);
    }
    const uint64_t prod = uint64_t(value) * uint64_t(int64_t(multiplier));
    const int64_t sum = int64_t(prod + uint64_t(round));
    return int32_t(uint32_t(uint64_t(sum >> (shift & 63))));
}

// One full RESCALE of a 32-bit-or-narrower value to a type with range [lo, hi]:
// subtract the input zero point, scale, add the output zero point (32-bit wrap), clamp.
__host__ __device__ inline int32_t rescaleValue(int64_t in, int32_t inZp, int32_t mult, int32_t shift,
                                                bool doubleRound, int32_t outZp, int32_t lo, int32_t hi) {
    int32_t r = applyScale(in - int64_t(inZp), mult, shift, doubleRound);
    r = int32_t(uint32_t(r) + uint32_t(outZp));
    return r < lo ? lo : (r > hi ? hi : r);
}

// ---- RESCALE in 32-bit-friendly form ---------------------------------------------------------------
// applyScale needs (v - zpIn) * mult + round in 64 bits, an arithmetic shift and a truncation to
// 32 bits.  With the input zero point folded into the rounding constant,
//     (v - zpIn) * mult + round  ==  v * mult + (round - zpIn * mult)      (mod 2^64)
// the whole step is one 32x32+64 multiply-add, one funnel shift and one shift.  The double-round
// variant adds +-2^30 by the sign of (v - zpIn), i.e. picks one of two constants by v >= zpIn.
// The low 32 bits of a 64-bit value shifted right by s are bits [s, s+32): for s <= 32 a funnel
// shift of the two halves, for s > 32 the high half shifted arithmetically by s - 32.
struct FastRescale {
    int32_t mult;
    int32_t zpIn;        // narrowed input zero point (threshold of the double-round sign test)
    uint32_t rpLo, rpHi; // rounding constant for v >= zpIn
    uint32_t rnLo, rnHi; // rounding constant for v <  zpIn
    int32_t s1, s2;      // min(shift, 32), max(shift - 32, 0)
};

__host__ __device__ inline FastRescale makeFastRescale(int32_t mult, int32_t shift, int32_t zpIn, bool doubleRound) {
    FastRescale f;
    shift = shift < 0 ? 0 : (shift > 62 ? 62 : shift); // other shifts are undefined in the reference shader
    uint64_t rp = shift > 0 ? (1ull << (shift - 1)) : 0ull;
    uint64_t rn = rp;
    if (doubleRound && shift > 31) {
        rp += 1ull << 30;
        rn -= 1ull << 30;
    }
    const uint64_t fold = uint64_t(0) - uint64_t(int64_t(zpIn)) * uint64_t(int64_t(mult));
    rp += fold;
    rn += fold;
    f.mult = mult;
    f.zpIn = zpIn;
    f.rpLo = uint32_t(rp), f.rpHi = uint32_t(rp >> 32);
    f.rnLo = uint32_t(rn), f.rnHi = uint32_t(rn >> 32);
    f.s1 = shift < 32 ? shift : 32;
    f.s2 = shift > 32 ? shift - 32 : 0;
    return f;
}

// int32(((int64(v) - zpIn) * mult + round) >> shift), bit-identical to applyScale.  The two rounding constants
// differ by 0 or 2^31, so the choice between them is the third input of the 64-bit addition that follows the
// multiply (one compare and one select) rather than a select of both halves of the constant.
__device__ __forceinline__ int32_t fastScale(int32_t v, int32_t mult, int32_t zpIn, uint32_t rpLo, uint32_t rpHi,
                                             uint32_t rnLo, uint32_t rnHi, int32_t s1, int32_t s2) {
    const uint64_t rn = (uint64_t(rnHi) << 32) | uint64_t(rnLo);
    const uint32_t bump = rpLo - rnLo; // (rp - rn) mod 2^32: 0 or 2^31
    const uint64_t sum = uint64_t(int64_t(v) * int64_t(mult)) + rn + uint64_t(v >= zpIn ? bump : 0u);
    const uint32_t t = __funnelshift_rc(uint32_t(sum), uint32_t(sum >> 32), uint32_t(s1));
    return int32_t(t) >> s2;
}

__device__ __forceinline__ int32_t fastRescale(const FastRescale &f, int32_t v, int32_t outZp, int32_t lo, int32_t hi) {
    int32_t r = fastScale(v, f.mult, f.zpIn, f.rpLo, f.rpHi, f.rnLo, f.rnHi, f.s1, f.s2);
    r = int32_t(uint32_t(r) + uint32_t(outZp));
    return min(max(r, lo), hi);
}

// High 32 bits of x * mult + round(x), x = value - input zero point: product and rounding of a RESCALE whose shift
// is at least 32, where the result only depends on the high word of the sum.  Double rounding adds 2^30 for x >= 0 and
// subtracts it for x < 0: that is rn = 2^(shift-1) - 2^30 plus 2^31 when the sign bit of x is clear, one logic
// operation on x (bumpMask = 2^31, or 0 without double rounding) feeding the third input of the 64-bit addition.
// (Measured and not kept: the same value as acc * mult + (corrX * mult + rn) with the bump and the remaining shift
// as multiply-high-adds.  It moves instructions from the general integer pipe to the multiply-add pipe, 56 % -> 43 %
// and 14 % -> 19 % of their peaks, and ran 10 % slower: this epilogue issues one instruction every other cycle
// whatever the mix.)
__device__ __forceinline__ int32_t scaleHigh(int32_t x, int32_t mult, uint64_t rn, uint32_t bumpMask) {
    const uint64_t prod = uint64_t(int64_t(x) * int64_t(mult));
    const uint32_t extra = ~uint32_t(x) & bumpMask;
    const uint64_t sum = prod + rn + uint64_t(extra);
    return int32_t(uint32_t(sum >> 32));
}

// The same RESCALE from 32-bit words only, for shifts of 32 to 60 and |x| < 2^29 (x = value - input zero point).
// Four times the sum is (4x) * mult + 2^(shift+1) +- 2^32: both rounding terms are whole units of the product's high
// word, and what the low word holds cannot change floor(sum / 2^shift) = (high + 2^(shift-31) +- 1) >> (shift - 30).
// x4 = 4x; c32 = 2^(shift-31), plus 1 with double rounding.  SIGNED: double rounding with the sign of x looked at
// (-1 instead of +1 for x < 0); callers leave it out where every x < 0 ends at the lower clamp bound either way.
template <bool SIGNED> __device__ __forceinline__ int32_t scaleHigh32(int32_t x4, int32_t mult, int32_t c32) {
    // (written out: from __mulhi(x4, mult) + c32 and + ((x4 >> 31) << 1) the compiler made a multiply-high, two
    // additions, a shift and a logic operation; counted over a ResNet-50 dispatch this form is 4 % fewer instructions)
    int32_t t;
    asm("mad.hi.s32 %0, %1, %2, %3;" : "=r"(t) : "r"(x4), "r"(mult), "r"(c32));
    if (SIGNED) {
        int32_t sign, u;
        asm("shr.s32 %0, %1, 31;" : "=r"(sign) : "r"(x4));
        asm("{\n\t.reg .s32 a;\n\tadd.s32 a, %1, %2;\n\tadd.s32 %0, a, %2;\n\t}" : "=r"(u) : "r"(t), "r"(sign));
        t = u;
    }
    return t;
}

} // namespace mlel
