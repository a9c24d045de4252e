// Device-side modular arithmetic for word-sized primes q < 2^61 (sm_100a).
// All helpers are exact: whichever reduction strategy a kernel uses (Shoup with a
// precomputed quotient, 128-bit Barrett, lazy ranges), stored results are the
// canonical residues in [0, q).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace hb {

using u32 = uint32_t;
using u64 = unsigned long long;
using i64 = long long;

constexpr int kMaxPrimes = 32;   // Q limbs + special limbs
constexpr int kMaxDigitLimbs = 8; // alpha upper bound
constexpr int kMaxList = 96;     // limb instances named by one launch

// Per-prime constants, one array per context in global memory.
struct PrimeConst {
    u64 q;
    u64 mu_hi, mu_lo;   // floor(2^128 / q)
    u64 n_inv, n_inv_sh; // N^-1 mod q and its Shoup companion
    u64 iu, iu_sh;      // psi^(N/2): the image of the imaginary unit
    u64 small;          // 1 when q < 2^44 and N = 2^16: the NTT tables hold w/q doubles (see mul_fp_lazy)
    double q_inv_f;     // 1/q
    double n_inv_f;     // n_inv / q
    u64 fp;             // 1 when q < 2^44: element-wise kernels take quotients from the FP64 pipe
    u64 lazy_terms;     // how many lazy products (each below 1.6 q) may be summed before the sum reaches 2^52
};

// Limb instances of a launch: instance li (0 <= li < count) uses prime[li % n].
struct LimbMap {
    int n;
    unsigned char prime[kMaxList];
};

__device__ __forceinline__ u64 mul_hi(u64 a, u64 b) { return __umul64hi(a, b); }

// x*w mod q in [0, 2q) for any x < 2^64, w < q, wsh = floor(w * 2^64 / q)
__device__ __forceinline__ u64 mul_shoup_lazy(u64 x, u64 w, u64 wsh, u64 q) {
    return x * w - mul_hi(x, wsh) * q;
}
__device__ __forceinline__ u64 mul_shoup(u64 x, u64 w, u64 wsh, u64 q) {
    u64 r = mul_shoup_lazy(x, w, wsh, q);
    return r >= q ? r - q : r;
}
// (z1:z0) mod q, any 128-bit input.  The quotient estimate is low by at most 4.
__device__ __forceinline__ u64 barrett128(u64 z1, u64 z0, const PrimeConst &m) {
    u64 qh = z1 * m.mu_hi + mul_hi(z1, m.mu_lo) + mul_hi(z0, m.mu_hi);
    u64 r = z0 - qh * m.q;
    u64 q4 = m.q << 2, q2 = m.q << 1;
    if (r >= q4) r -= q4;
    if (r >= q2) r -= q2;
    if (r >= m.q) r -= m.q;
    return r;
}
__device__ __forceinline__ u64 mul_mod(u64 a, u64 b, const PrimeConst &m) {
    return barrett128(mul_hi(a, b), a * b, m);
}
__device__ __forceinline__ u64 add_mod(u64 a, u64 b, u64 q) { u64 s = a + b; return s >= q ? s - q : s; }
__device__ __forceinline__ u64 sub_mod(u64 a, u64 b, u64 q) { return a >= b ? a - b : a + q - b; }
__device__ __forceinline__ u64 reduce_u64(u64 x, const PrimeConst &m) { return barrett128(0, x, m); }
__device__ __forceinline__ u64 reduce_i64(i64 v, const PrimeConst &m) {
    if (v >= 0) return reduce_u64((u64)v, m);
    u64 r = reduce_u64((u64)(-(v + 1)), m);
    return m.q - 1 - r;
}
// ---- FP64-assisted product for primes below 2^44 ------------------------------------------
// B200 issues 64-bit integer adds, compares and selects on a half-rate ALU pipe, and that pipe is
// what bounds a Shoup butterfly (17 ALU instructions each).  For small primes the quotient
// floor(y*w/q) is taken from the FP64 pipe instead: y < 2^52 converts exactly through the 2^52
// magic constant, fma(y, w/q, 2^52) leaves round(y*w/q) in the mantissa (error well below 1),
// and the remainder y*w - qh*q is exact in 64-bit integer arithmetic.  The result is congruent
// to y*w and lies in (0.4q, 1.6q); final stores reduce to the canonical residue, so the bits
// that reach memory are those of any other exact method.
constexpr double kTwo52 = 4503599627370496.0;
__device__ __forceinline__ double u52_to_double(u64 v) { return __longlong_as_double((long long)(v | 0x4330000000000000ull)) - kTwo52; }
__device__ __forceinline__ u64 mantissa52(double d) { return (u64)__double_as_longlong(d) & 0x000FFFFFFFFFFFFFull; }
// low 64 bits of a*b + c*d + e as one chain of integer multiply-adds (no separate add instructions)
__device__ __forceinline__ u64 mad2_lo64(u64 a, u64 b, u64 c, u64 d, u64 e) {
    const u32 a0 = (u32)a, a1 = (u32)(a >> 32), b0 = (u32)b, b1 = (u32)(b >> 32);
    const u32 c0 = (u32)c, c1 = (u32)(c >> 32), d0 = (u32)d, d1 = (u32)(d >> 32);
    u64 r;
    asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(r) : "r"(a0), "r"(b0), "l"(e));
    asm("mad.wide.u32 %0, %1, %2, %0;" : "+l"(r) : "r"(c0), "r"(d0));
    u32 lo = (u32)r, hi = (u32)(r >> 32);
    asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(hi) : "r"(a0), "r"(b1));
    asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(hi) : "r"(a1), "r"(b0));
    asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(hi) : "r"(c0), "r"(d1));
    asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(hi) : "r"(c1), "r"(d0));
    return ((u64)hi << 32) | lo;
}
__device__ __forceinline__ u64 mul_fp_lazy(u64 y, u64 w, double w_over_q, u64 q) {
    const u64 qh = mantissa52(__fma_rn(u52_to_double(y), w_over_q, kTwo52));
    return mad2_lo64(y, w, qh, 0ull - q, q); // y*w - qh*q + q
}
// v < 2^52 -> residue in (0.4q, 1.6q)
__device__ __forceinline__ u64 reduce_fp_lazy(u64 v, double q_inv, u64 q) {
    const u64 qh = mantissa52(__fma_rn(u52_to_double(v), q_inv, kTwo52));
    return v - qh * q + q;
}
// v < 2^52 -> canonical residue
__device__ __forceinline__ u64 reduce_fp(u64 v, double q_inv, u64 q) {
    const u64 r = reduce_fp_lazy(v, q_inv, q); // (0.4q, 1.6q)
    return r >= q ? r - q : r;
}

// a*b for a, b < 2^44 and q < 2^44: result congruent to a*b in (0.4q, 1.6q).  The double product is only
// used for the quotient estimate (relative error 2^-52, far below one unit); the remainder is exact.
__device__ __forceinline__ u64 mul_small_lazy_d(u64 a, double ad, u64 b, double bd, double q_inv, u64 q) {
    const u64 qh = mantissa52(__fma_rn(ad * bd, q_inv, kTwo52));
    return mad2_lo64(a, b, qh, 0ull - q, q);
}
__device__ __forceinline__ u64 mul_small_lazy(u64 a, u64 b, double q_inv, u64 q) {
    return mul_small_lazy_d(a, u52_to_double(a), b, u52_to_double(b), q_inv, q);
}
// canonical a*b mod q, choosing the FP64-assisted form for small primes
__device__ __forceinline__ u64 mul_mod_any(u64 a, u64 b, const PrimeConst &m) {
    if (m.fp) { const u64 r = mul_small_lazy(a, b, m.q_inv_f, m.q); return r >= m.q ? r - m.q : r; }
    return mul_mod(a, b, m);
}
// canonical residue of a signed value
__device__ __forceinline__ u64 reduce_i64_any(i64 v, const PrimeConst &m) {
    const u64 a = v < 0 ? (u64)(-(v + 1)) + 1 : (u64)v;
    if (m.fp && a < (1ull << 51)) {
        u64 r = reduce_fp(a, m.q_inv_f, m.q);
        return (v < 0 && r) ? m.q - r : r;
    }
    return reduce_i64(v, m);
}

// ---- the product of two residues of a prime below 2^44 entirely on the FP64 pipe ---------------------------------
// a, w: integer-valued doubles, |a| < 2^44, |w| < 2^44.  p + e = a * w exactly (rounded product and its error, one FMA),
// the quotient estimate rint(p / q) is off by far less than one, p - qh * q is an integer below 2^45 and so is its sum
// with e: the result is congruent to a * w and lies within 0.51 q of zero.  Seven FP64 instructions with the running
// sum, no conversions, against about eleven mixed ones for the integer-assisted form.
constexpr double kMagicS = 6755399441055744.0; // 2^52 + 2^51
__device__ __forceinline__ double mul_fp64_lazy(double a, double w, double q_inv, double qd) {
    const double p = __dmul_rn(a, w);
    const double e = __fma_rn(a, w, -p);
    const double qh = __dadd_rn(__fma_rn(p, q_inv, kMagicS), -kMagicS);
    return __dadd_rn(__fma_rn(-qh, qd, p), e);
}
// integer-valued double, |v| < 2^50  ->  canonical residue in [0, q)
__device__ __forceinline__ u64 canon_fp64(double v, double q_inv, double qd) {
    const double k = __dadd_rn(__fma_rn(v, q_inv, kMagicS), -kMagicS);
    double r = __fma_rn(-k, qd, v);        // within 0.51 q of zero, exact
    if (r < 0.0) r = __dadd_rn(r, qd);
    return mantissa52(__dadd_rn(r, kTwo52));
}

// 128-bit accumulator for lazy sums of products
struct Acc128 {
    u64 lo, hi;
    __device__ __forceinline__ void zero() { lo = 0; hi = 0; }
    __device__ __forceinline__ void mad(u64 a, u64 b) {
        u64 pl = a * b, ph = mul_hi(a, b);
        lo += pl; hi += ph + (lo < pl);
    }
};

// ---- sums of products modulo the primes of 44 to 60 bits ---------------------------------------------------------
// A full 64 x 64 -> 128-bit product with its carries costs about thirty 32-bit multiply-adds on this GPU.  For lazy
// sums of a few products the operands are cut into two pieces of 30 bits instead: a product is then four
// 32 x 32 -> 64-bit multiply-adds, one per pair of pieces, each into its own 64-bit accumulator with no carries, and
// the sum of products is  a0 + (a1 + a2) * 2^30 + a3 * 2^60,  assembled and reduced once per output residue.
// A piece product is below 2^60, so an accumulator holds 16 terms; flush() folds them into a 128-bit running sum.
__device__ __forceinline__ u64 mad_wide(u32 a, u32 b, u64 c) {
    u64 r;
    asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(r) : "r"(a), "r"(b), "l"(c));
    return r;
}
struct PieceAcc {
    u64 a0, a1, a2, a3, lo, hi;
    __device__ __forceinline__ void zero() { a0 = a1 = a2 = a3 = 0; lo = hi = 0; }
    __device__ __forceinline__ void mac(u64 v, u64 k) { // v, k < 2^60
        const u32 v0 = (u32)v & 0x3FFFFFFFu, v1 = (u32)(v >> 30), k0 = (u32)k & 0x3FFFFFFFu, k1 = (u32)(k >> 30);
        a0 = mad_wide(v0, k0, a0); a1 = mad_wide(v0, k1, a1); a2 = mad_wide(v1, k0, a2); a3 = mad_wide(v1, k1, a3);
    }
    __device__ __forceinline__ void add128(u64 l, u64 h) { lo += l; hi += h + (lo < l); }
    __device__ __forceinline__ void flush() {
        add128(a0, 0);
        add128(a1 << 30, a1 >> 34);
        add128(a2 << 30, a2 >> 34);
        add128(a3 << 60, a3 >> 4);
        a0 = a1 = a2 = a3 = 0;
    }
    __device__ __forceinline__ u64 finish(const PrimeConst &m) { flush(); return barrett128(hi, lo, m); }
};

// index of the source slot of the automorphism X -> X^g on an NTT-form limb:
//   out[i] = in[ntt_perm(i)], exponents 2*bitrev(i)+1 multiply by g modulo 2N
__device__ __forceinline__ u32 ntt_perm(u32 i, u32 g, int logn) {
    u32 e = ((__brev(i) >> (32 - logn)) << 1) | 1u;
    u32 ej = (g * e) & ((2u << logn) - 1u);
    return __brev(ej >> 1) >> (32 - logn);
}

} // namespace hb
