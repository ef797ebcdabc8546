// Shared host/device definitions of librns_b200: error plumbing, the host-side
// number theory that turns a modulus list into kernel constants, and the
// per-element reconstruction arithmetic used by every epilogue.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>
#include <cstring>

#include "../../include/rns_b200.h"

namespace rns {

// ---------------------------------------------------------------------------
// Errors
// ---------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);

#define RNS_CUDA_OK(expr)                                                        \
    do {                                                                         \
        cudaError_t err__ = (expr);                                              \
        if (err__ != cudaSuccess)                                                \
            return ::rns::fail(RNS_ERR_CUDA, "%s failed: %s", #expr,             \
                               cudaGetErrorString(err__));                       \
    } while (0)

// ---------------------------------------------------------------------------
// Constants of one modulus set, as kernels consume them (passed by value in
// kernel parameters, so every access with a compile-time index is a constant
// bank operand).
// ---------------------------------------------------------------------------
constexpr int kMaxCh = RNS_MAX_CHANNELS;

struct Plan {
    int32_t channels;
    int32_t mod[kMaxCh];
    // floor(2^32/m) clipped to INT32_MAX: q = mulhi(v, recip) is within one of
    // floor(v/m) for any int32 v, so v - q*m lies in [-m, 2m).
    int32_t recip[kMaxCh];
    // m * floor(2^31 / m): added to an int32 sum it gives a non-negative uint32 of the same
    // residue class (needs |sum| <= 2^31 - m, which the K bound of the callers guarantees).
    uint32_t ubias[kMaxCh];
    float modf[kMaxCh];
    float rcpf[kMaxCh];            // 1.0f / m
    // Flattened Garner: digit_i = centred( r_i*gscale[i] + sum_{j<i} gneg[i][j]*digit_j  mod m_i )
    // with gscale[i] = (m_0..m_{i-1})^-1 mod m_i and gneg[i][j] = -(m_0..m_{j-1}) * gscale[i]
    // mod m_i, both stored as centred representatives.  Every partial sum stays
    // below 2^24 in magnitude (|r| < 2m, |digit| <= m/2, m <= 255, <= 10 terms),
    // so fp32 evaluates it exactly.
    float gscale[kMaxCh];
    float gneg[kMaxCh][kMaxCh];
    // Place values prod_{t<i} m_t.  The first four always fit 32 bits together
    // with the centred partial sum they build (255^4/2 < 2^31).
    uint32_t place32[4];
    int64_t place64[kMaxCh];
    int64_t product[kMaxCh + 1];   // product[c] = m_0*...*m_{c-1}; product[0] = 1
    // SWAR encoder constants (valid when encode_single_fold): bytes of
    // enc_hi = 127 - floor(m/2), enc_lo = floor(m/2), replicated four times.
    uint32_t enc_hi[kMaxCh];
    uint32_t enc_lo[kMaxCh];
    uint32_t enc_mk[kMaxCh];       // m << 25 when encode_fast, else m
    int32_t encode_fast;           // every modulus < 128
    uint32_t enc_mfold[kMaxCh];    // reduced encoder: m if m <= 191 else 0
    int32_t encode_single_fold;    // every modulus >= 86
};

// Packed tile layouts (see rns_linear_args in the public header).
constexpr int kPackK = 64;     // bytes of K per packed row
constexpr int kPackM = 128;    // activation rows per packed tile
constexpr int kPackNPad = 384; // weight rows are padded to a multiple of this

#ifdef __CUDACC__
#define RNS_HD_INLINE __host__ __device__ __forceinline__
#else
#define RNS_HD_INLINE inline
#endif
RNS_HD_INLINE int64_t round_up_i64(int64_t v, int64_t q) { return (v + q - 1) / q * q; }
// Offset inside one [rows][64] packed block of byte `col` (0..63) of row `row`.
RNS_HD_INLINE int packed_row_offset(int row, int col) {
    return row * kPackK + ((((col >> 4) ^ ((row >> 1) & 3)) << 4) | (col & 15));
}
// Weight byte (n, k) -> offset in [K_pad/64][N_pad][64].
RNS_HD_INLINE int64_t packed_weight_offset(int n, int k, int64_t n_pad) {
    return ((int64_t)(k >> 6) * n_pad) * kPackK + packed_row_offset(n, k & 63);
}
// Activation byte (m, k) of channel c -> offset in [M_pad/128][K_pad/64][channels][128][64].
RNS_HD_INLINE int64_t packed_act_offset(int m, int k, int c, int channels, int64_t kblocks) {
    const int64_t tile = ((int64_t)(m >> 7) * kblocks + (k >> 6)) * channels + c;
    return tile * (kPackM * kPackK) + packed_row_offset(m & 127, k & 63);
}

// Builds the plan; returns an rns_status.  Pure host arithmetic.
int build_plan(const int32_t* moduli, int channels, Plan* out);

// ---------------------------------------------------------------------------
// Device arithmetic shared by the epilogues
// ---------------------------------------------------------------------------
#ifdef __CUDACC__
#define RNS_HD __host__ __device__ __forceinline__
#else
#define RNS_HD inline
#endif

// The arithmetic below compiles for the host as well, so that CPU tests can run
// the exact expressions the kernels evaluate.
constexpr float kMagic = 12582912.0f;          // 1.5 * 2^23
constexpr int kMagicBits = 0x4B400000;

RNS_HD float bits_to_float(int v) {
#ifdef __CUDA_ARCH__
    return __int_as_float(v);
#else
    float f; memcpy(&f, &v, 4); return f;
#endif
}
RNS_HD int float_to_bits(float f) {
#ifdef __CUDA_ARCH__
    return __float_as_int(f);
#else
    int v; memcpy(&v, &f, 4); return v;
#endif
}
RNS_HD float fma_rn(float a, float b, float c) {
#ifdef __CUDA_ARCH__
    return __fmaf_rn(a, b, c);
#else
    return __builtin_fmaf(a, b, c);
#endif
}
RNS_HD float mul_rn(float a, float b) {
#ifdef __CUDA_ARCH__
    return __fmul_rn(a, b);
#else
    volatile float r = a * b; return r;
#endif
}
RNS_HD float add_rn(float a, float b) {
#ifdef __CUDA_ARCH__
    return __fadd_rn(a, b);
#else
    volatile float r = a + b; return r;
#endif
}
RNS_HD int mul_hi(int a, int b) {
#ifdef __CUDA_ARCH__
    return __mulhi(a, b);
#else
    return (int)(((long long)a * (long long)b) >> 32);
#endif
}
RNS_HD uint32_t mul_hi_u32(uint32_t a, uint32_t b) {
#ifdef __CUDA_ARCH__
    return __umulhi(a, b);
#else
    return (uint32_t)(((unsigned long long)a * (unsigned long long)b) >> 32);
#endif
}

// Exact int -> float for |v| < 2^22 without the conversion unit.
RNS_HD float small_int_to_float(int v) { return add_rn(bits_to_float(v + kMagicBits), -kMagic); }
// Exact float (integral, |v| < 2^22) -> int.
RNS_HD int small_float_to_int(float v) { return float_to_bits(add_rn(v, kMagic)) - kMagicBits; }

// Loose residue of an int32 accumulator: congruent to v mod m, in [-m, 2m).
RNS_HD int loose_residue(int v, int m, int recip) { return v - mul_hi(v, recip) * m; }

// Canonical residue in [0, m) of an int32 accumulator with |v| <= 2^31 - m: bias to a
// non-negative uint32, unsigned Barrett step (quotient at most one short), one conditional
// subtraction.  Fits a byte for every modulus up to 255.
RNS_HD uint32_t canonical_residue(int v, int m, int recip, uint32_t ubias) {
    const uint32_t u = (uint32_t)v + ubias;
    uint32_t r = u - mul_hi_u32(u, (uint32_t)recip) * (uint32_t)m;      // [0, 2m)
    const uint32_t r2 = r - (uint32_t)m;
    return r2 < r ? r2 : r;                                             // r >= m: r - m, else r
}

// The same without the conditional subtraction: a residue in [0, 2m), which still fits a byte
// when m <= 127.
RNS_HD uint32_t nonneg_residue(int v, int m, int recip, uint32_t ubias) {
    const uint32_t u = (uint32_t)v + ubias;
    return u - mul_hi_u32(u, (uint32_t)recip) * (uint32_t)m;
}

// t -> representative of t mod m with |result| <= m/2 (t integral, |t| < 2^22).
RNS_HD float centre_mod(float t, float m, float rcp) {
    const float q = add_rn(fma_rn(t, rcp, kMagic), -kMagic);
    return fma_rn(-q, m, t);
}

// Centred digits of the mixed-radix form of the value whose channel sums are acc[].
template <int R>
RNS_HD void garner_digits(const int (&acc)[R], const Plan& pl, int active, float (&digit)[R]) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
        digit[i] = 0.0f;
        if (i < active) {
            const float r = small_int_to_float(loose_residue(acc[i], pl.mod[i], pl.recip[i]));
            float t = (i == 0) ? r : mul_rn(r, pl.gscale[i]);
#pragma unroll
            for (int j = 0; j < i; ++j) t = fma_rn(pl.gneg[i][j], digit[j], t);
            digit[i] = centre_mod(t, pl.modf[i], pl.rcpf[i]);
        }
    }
}

// Mixed-radix reconstruction of one output element from R int32 channel sums.
// Follows csrc/rns_cuda.cu:380-414 of the reference (digits, place-value sum,
// "if x > P/2: x -= P") but with centred digits, so the sum is already signed;
// the final range fix-up reproduces the reference's representative (-P/2, P/2]
// in every case, including even P and inputs beyond the capacity.
// Returns the value as int64; `active` (<= R) is the number of channels in use.
template <int R>
RNS_HD long long reconstruct(const int (&acc)[R], const Plan& pl, int active) {
    float digit[R];
    garner_digits<R>(acc, pl, active, digit);
    int lo = 0;
#pragma unroll
    for (int i = 0; i < (R < 4 ? R : 4); ++i)
        if (i < active) lo += (int)pl.place32[i] * small_float_to_int(digit[i]);
    long long x = lo;
    if (R > 4) {
#pragma unroll
        for (int i = 4; i < R; ++i)
            if (i < active) x += pl.place64[i] * (long long)small_float_to_int(digit[i]);
    }
    const long long prod = pl.product[active];
    const long long half = prod >> 1;
    if (x > half) x -= prod;
    else if (x < half - prod + 1) x += prod;
    return x;
}

// Same, for R <= 4 where everything fits 32 bits (P < 2^32, |x| <= P/2 < 2^31).
template <int R>
RNS_HD int reconstruct32(const int (&acc)[R], const Plan& pl, int active) {
    static_assert(R <= 4, "32-bit reconstruction covers at most four channels");
    float digit[R];
    garner_digits<R>(acc, pl, active, digit);
    unsigned x = 0;
    if (R == 4 && active == 4) {
        // d0 + m0*d1 and d2 + m2*d3 are exact in fp32 (|.| < 2^15): two conversions and
        // one integer multiply-add instead of four of each.
        const float lo = fma_rn(pl.modf[0], digit[1], digit[0]);
        const float hi = fma_rn(pl.modf[R > 2 ? 2 : 0], digit[R > 3 ? 3 : 0], digit[R > 2 ? 2 : 0]);
        x = (unsigned)small_float_to_int(lo) + pl.place32[R > 2 ? 2 : 0] * (unsigned)small_float_to_int(hi);
    } else {
#pragma unroll
        for (int i = 0; i < R; ++i)
            if (i < active) x += pl.place32[i] * (unsigned)small_float_to_int(digit[i]);
    }
    const unsigned prod = (unsigned)pl.product[active];
    const int half = (int)(prod >> 1);
    const int low = (int)((unsigned)half - prod + 1u);
    int sx = (int)x;
    if (sx > half) sx = (int)(x - prod);
    else if (sx < low) sx = (int)(x + prod);
    return sx;
}


// Centred residues of four packed int8 values for one modulus (single fold;
// requires m >= 86).  u = bytes biased by 128, ul = u with the top bit of each
// byte cleared, hi/lo = Plan::enc_hi/enc_lo.  Bit 7 of (ul + hi) & u is set
// where x > floor(m/2); bit 7 of ~((ul + lo) | u) where x < -floor(m/2).  The
// biased result never leaves [0,255] per byte, so 32-bit arithmetic applies all
// four folds without carries between bytes.  -m/2 of an even modulus is kept
// negative, as the reference's device encoder does (csrc/rns_cuda.cu:116-122).
//
// Two forms of the last step.  FAST (every modulus < 128, mk = m << 25):
// mulhi(mask, mk) turns each set bit 8i+7 into m << 8i; the multiplies run on
// the FMA pipe and leave the integer ALU (half rate on this architecture) the
// two logic operations.  Otherwise the masks are shifted down and multiplied by
// m (mk = m).
template <bool FAST>
RNS_HD uint32_t encode_word(uint32_t u, uint32_t ul, uint32_t hi, uint32_t lo, uint32_t mk) {
    const uint32_t down = (ul + hi) & u & 0x80808080u;
    const uint32_t up = ~((ul + lo) | u) & 0x80808080u;
    uint32_t v;
    if (FAST) v = mul_hi_u32(up, mk) + u - mul_hi_u32(down, mk);
    else v = u + ((up >> 7) - (down >> 7)) * mk;
    return v ^ 0x80808080u;
}

// One-step reduced residues of four packed int8 values, the default encoder of
// the fused kernel.  A value is folded once, towards zero, when its two top bits
// differ (x >= 64 or x < -64):  r = x - m for x >= 64,  r = x + m for x < -64,
// r = x otherwise, for every modulus m <= 191 (larger moduli, whose residues of
// int8 values need no fold below 96, pass through: mfold = 0).  r is congruent to
// x and fits a signed byte for every modulus in [2,255]; for the moduli just
// below 128 it is the centred residue except within a few units of +-64
// (|r| <= 64 instead of <= m/2), which is all the int32 accumulation and the
// reconstruction need.  The fold pattern does not depend on the modulus, so it
// is computed once per word (fold_pattern) and each channel costs one
// multiply-add and one xor.
//   u = x ^ 0x80808080 (bytes biased by 128);  d = per-byte +1 / -1 / 0 pattern
RNS_HD uint32_t fold_pattern(uint32_t x) {
    const uint32_t f = (x ^ (x << 1)) & 0x80808080u;   // bit 7: top two bits differ
    const uint32_t up = f & x;                          // negative: add m
    return (up >> 6) - (f >> 7);                        // 2*up7 - f7 = up7 - down7
}
RNS_HD uint32_t encode_word_reduced(uint32_t u, uint32_t d, uint32_t mfold) {
    return (u + d * mfold) ^ 0x80808080u;
}

}  // namespace rns
