// Negacyclic NTT / inverse NTT of 2^16-coefficient limbs for sm_100a.
//
// Output order of the forward transform: a_hat[i] = a(psi^(2*bitrev(i)+1)) -- the order of the tables psi^bitrev(k).
//
// The limb is a 256 x 256 matrix (index = row*256 + col).  The forward transform is a column pass (stages 1-8,
// butterfly distance >= 256) followed by a row pass (stages 9-16); the inverse runs the row pass first.  A pass moves
// a limb through HBM once: a CTA of 256 threads owns 16 columns (or 16 rows), every thread keeps 16 coefficients in
// registers and performs four butterfly stages at a time (radix 16), exchanging through shared memory once.
//
// Two things set these kernels apart from a textbook radix-2 transform:
//
//  * Twiddles are stored in the order the kernels read them (Ntt16Layout): 16-byte entries (w, companion) so that one
//    128-bit load fetches both words, at offsets that are compile-time constants from one per-thread base pointer.
//    The 15 twiddles a thread owns alone in the last four stages sit 16 entries apart, so the 16 threads of a row
//    read 256 contiguous bytes per load.
//
//  * For primes below 2^44 the coefficients are carried as integer-valued doubles ("double storage") from the first
//    load of a transform to its last store, signed and unreduced.  A butterfly is then
//        qh = fma(y, w/q, M)                 quotient estimate, M = 2^52 + 2^51          (FP64)
//        yb = y + M                          integer image of y in the mantissa           (FP64)
//        r  = yb*w - qh*q + q  (low 48 bits)  six 32-bit multiply-adds                     (FMA pipe)
//        t  = double(2^52 | r) - (2^52 + q)  exact remainder in (-0.52 q, 0.52 q)          (1 logic op + FP64)
//        x' = x + t,  y' = x - t                                                          (FP64)
//    twelve instructions, five of them on the FP64 pipe, six on the multiply-add pipe and one on the ALU, where the
//    all-integer butterfly spends most of its issue slots on 64-bit adds, compares and selects.  Every step is exact:
//    the quotient estimate is off by less than 0.02, so the remainder is the true residue class representative in
//    (-0.52 q, 0.52 q); values grow by at most 0.52 q per forward stage (|x| < 9.4 q after 16 stages, far below 2^51).
//    The pass boundary stores the doubles as they are (the intermediate array is private to the transform); the last
//    store reduces to the canonical residue, so the bits that reach memory are those of any other exact method.
//    Primes of 44 bits and more use Shoup butterflies on integers in [0, 4q).
#pragma once
#include "modarith.cuh"
#include <cstring>

namespace hb {

constexpr int kN16 = 65536;
constexpr int kRowStride = 272; // 256 + one pad word per 16: conflict-free 16-consecutive reads

// Where twiddle psi^bitrev((base << s) + g) of a four-stage round sits in the per-prime table; j = (1 << s) - 1 + g.
struct Ntt16Layout {
    static constexpr int kColsA = 0;                // column pass, first round: base 1, shared by everybody
    static constexpr int kColsB = 16;               // column pass, second round: base 16 + sub, 16 entries per sub
    static constexpr int kRowsA = 16 + 16 * 16;     // row pass, first round: base 256 + row, 16 entries per row
    static constexpr int kRowsB = kRowsA + 256 * 16; // row pass, second round: base (256 + row) * 16 + clo, entry j of lane clo at (row * 15 + j) * 16 + clo
    static constexpr int kEntries = kRowsB + 256 * 15 * 16;
    static __host__ __device__ constexpr int colsA(int j) { return kColsA + j; }
    static __host__ __device__ constexpr int colsB(int sub, int j) { return kColsB + sub * 16 + j; }
    static __host__ __device__ constexpr int rowsA(int row, int j) { return kRowsA + row * 16 + j; }
    static __host__ __device__ constexpr int rowsB(int row, int j, int clo) { return kRowsB + (row * 15 + j) * 16 + clo; }
};
// entry: x = w, y = companion (bits of the double w/q for primes below 2^44, Shoup quotient otherwise)
struct Ntt16Tables {
    const ulonglong2 *fwd, *inv; // each [nprimes][Ntt16Layout::kEntries]
    // the last round of the row pass for primes below 2^44: the twiddle alone as a double, [nprimes][kRowsB8], entry j of
    // lane clo of row `row` at (row * 15 + j) * 16 + clo -- half the bytes of the 16-byte entries, and in that round every
    // thread reads 15 twiddles nobody else uses (more bytes than the coefficients themselves)
    const double *fwdB8, *invB8;
};
constexpr int kRowsB8 = 256 * 15 * 16;

// Fills one prime's table from psi^bitrev(k) (k < 2^16) and the companion words; host side.
template <class F> inline void ntt16_fill_table(ulonglong2 *out, F entry /* (index into the bit-reversed table) -> ulonglong2 */) {
    auto put = [&](int off, unsigned base) {
        for (int s = 0; s < 4; ++s)
            for (int g = 0; g < (1 << s); ++g) out[off + (1 << s) - 1 + g] = entry((base << s) + (unsigned)g);
    };
    put(Ntt16Layout::colsA(0), 1u);
    for (int sub = 0; sub < 16; ++sub) put(Ntt16Layout::colsB(sub, 0), 16u + (unsigned)sub);
    for (int row = 0; row < 256; ++row) put(Ntt16Layout::rowsA(row, 0), 256u + (unsigned)row);
    for (int row = 0; row < 256; ++row)
        for (int clo = 0; clo < 16; ++clo) {
            const unsigned base = ((256u + (unsigned)row) << 4) + (unsigned)clo;
            for (int s = 0; s < 4; ++s)
                for (int g = 0; g < (1 << s); ++g) out[Ntt16Layout::rowsB(row, (1 << s) - 1 + g, clo)] = entry((base << s) + (unsigned)g);
        }
}

// the compact last-round table of one prime below 2^44: w(k) = the twiddle of bit-reversed-table index k as a double
template <class F> inline void ntt16_fill_rows_b8(double *out, F w) {
    for (int row = 0; row < 256; ++row)
        for (int clo = 0; clo < 16; ++clo) {
            const unsigned base = ((256u + (unsigned)row) << 4) + (unsigned)clo;
            for (int s = 0; s < 4; ++s)
                for (int g = 0; g < (1 << s); ++g) out[(row * 15 + (1 << s) - 1 + g) * 16 + clo] = w((base << s) + (unsigned)g);
        }
}

// Optional last multiplication of the inverse transform: position k = li % map.n gets scale s_k (which must already
// contain N^-1) instead of N^-1 -- a base conversion that follows folds its first product (the inverse of a complementary
// modulus) into the transform.  w: s_k (as ds_twiddle_word for primes below 2^44), comp: s_k / q as a double, or the
// Shoup companion.
struct Ntt16Scale { u64 w[8], comp[8]; int on; };

// address of limb instance li: (li / period) * outer + (li % period) * N
struct LimbAddr16 {
    size_t outer;
    __device__ __forceinline__ size_t off(int li, int period) const { return (size_t)(li / period) * outer + (size_t)(li % period) * kN16; }
};

// ---------------- Shoup butterflies on integers (primes of 44 bits and more) ----------------
__device__ __forceinline__ void ct_bfly(u64 &x, u64 &y, u64 w, u64 ws, u64 q, u64 q2) {
    x = x >= q2 ? x - q2 : x;
    u64 t = mul_shoup_lazy(y, w, ws, q);
    y = x + q2 - t;
    x = x + t;
}
__device__ __forceinline__ void gs_bfly(u64 &x, u64 &y, u64 w, u64 ws, u64 q, u64 q2) {
    u64 s = x + y;
    u64 d = x + q2 - y;
    x = s >= q2 ? s - q2 : s;
    y = mul_shoup_lazy(d, w, ws, q);
}
// four Cooley-Tukey stages on 16 register values; twiddle j = (1 << s) - 1 + g of local stage s, group g, at tp[j * STRIDE]
template <int STRIDE> __device__ __forceinline__ void fwd16_int(u64 (&v)[16], const ulonglong2 *__restrict__ tp, u64 q) {
    const u64 q2 = q << 1;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        const int half = 8 >> s;
#pragma unroll
        for (int g = 0; g < (1 << s); ++g) {
            const ulonglong2 tw = __ldg(tp + ((1 << s) - 1 + g) * STRIDE);
#pragma unroll
            for (int j = 0; j < half; ++j) ct_bfly(v[g * 2 * half + j], v[g * 2 * half + j + half], tw.x, tw.y, q, q2);
        }
    }
}
// four Gentleman-Sande stages, the mirror image
template <int STRIDE> __device__ __forceinline__ void inv16_int(u64 (&v)[16], const ulonglong2 *__restrict__ tp, u64 q) {
    const u64 q2 = q << 1;
#pragma unroll
    for (int s = 3; s >= 0; --s) {
        const int half = 8 >> s;
#pragma unroll
        for (int g = 0; g < (1 << s); ++g) {
            const ulonglong2 tw = __ldg(tp + ((1 << s) - 1 + g) * STRIDE);
#pragma unroll
            for (int j = 0; j < half; ++j) gs_bfly(v[g * 2 * half + j], v[g * 2 * half + j + half], tw.x, tw.y, q, q2);
        }
    }
}

// ---------------- double-storage butterflies (primes below 2^44) ----------------
constexpr double kMagic = 6755399441055744.0; // 2^52 + 2^51: adding it leaves a signed integer |v| < 2^51 in the low mantissa bits
struct DsConst {
    u64 nq;      // 2^64 - q
    u64 q;
    double coff; // 2^52 + q
    double qd, qinv;
};
__device__ __forceinline__ DsConst ds_const(const PrimeConst &m) {
    DsConst c;
    c.nq = 0ull - m.q; c.q = m.q; c.coff = kTwo52 + (double)m.q; c.qd = (double)m.q; c.qinv = m.q_inv_f;
    return c;
}
// canonical residue -> double, exact for values below 2^52
__device__ __forceinline__ double ds_load(u64 a) { return u52_to_double(a); }
// t = y * w mod q as a signed double in (-0.52 q, 0.52 q); y integer-valued, |y| < 2^49; wf = w / q
#ifndef HB_DS_FP
#define HB_DS_FP 1
#endif
#if HB_DS_FP
// wbits = bits of the double w.  Six FP64 instructions, every one exact: p + e = y * w (product and its rounding error),
// qh = rint(y * w / q) up to 0.02, p - qh * q is an integer below 2^45 and so is its sum with e.
__device__ __forceinline__ double ds_mul(double y, u64 wbits, double wf, const DsConst &c) {
    const double wd = __longlong_as_double((long long)wbits);
    const double qh = __dadd_rn(__fma_rn(y, wf, kMagic), -kMagic);
    const double p = __dmul_rn(y, wd);
    const double e = __fma_rn(y, wd, -p);
    const double t1 = __fma_rn(-qh, c.qd, p);
    return __dadd_rn(t1, e);
}
#else
__device__ __forceinline__ double ds_mul(double y, u64 w, double wf, const DsConst &c) {
    const double qh = __fma_rn(y, wf, kMagic);
    const double yb = __dadd_rn(y, kMagic);
    const u64 r = mad2_lo64((u64)__double_as_longlong(yb), w, (u64)__double_as_longlong(qh), c.nq, c.q); // y*w - qh*q + q, exact in its low 48 bits
    const u32 hi = ((u32)(r >> 32) & 0xFFFFu) | 0x43300000u;
    return __hiloint2double((int)hi, (int)(u32)r) - c.coff;
}
#endif
// the same with the quotient estimated from the rounded product instead of from a precomputed w / q (one operand less to
// fetch; the estimate is off by less than 0.07, so the result lies within 0.57 q of zero)
__device__ __forceinline__ double ds_mul_w(double y, double wd, const DsConst &c) {
    const double p = __dmul_rn(y, wd);
    const double e = __fma_rn(y, wd, -p);
    const double qh = __dadd_rn(__fma_rn(p, c.qinv, kMagic), -kMagic);
    return __dadd_rn(__fma_rn(-qh, c.qd, p), e);
}
// the form of a twiddle w that ds_mul takes as its second operand
__host__ __device__ __forceinline__ u64 ds_twiddle_word(u64 w) {
#if HB_DS_FP
    const double d = (double)w; // exact below 2^53
#ifdef __CUDA_ARCH__
    return (u64)__double_as_longlong(d);
#else
    u64 b; memcpy(&b, &d, 8); return b;
#endif
#else
    return w;
#endif
}
// x - rint(x / q) * q, |result| <= 0.52 q
__device__ __forceinline__ double ds_reduce(double x, const DsConst &c) {
    const double k = __fma_rn(x, c.qinv, kMagic) - kMagic;
    return __fma_rn(-k, c.qd, x);
}
// integer-valued double, |v| < 2^20 q  ->  canonical residue in [0, q)
__device__ __forceinline__ u64 ds_store(double v, const DsConst &c, double shift /* a multiple of q above |v| */, double qinv_up) {
    const double v2 = v + shift;                                         // positive
    const double k = __fma_rd(v2, qinv_up, kTwo52) - kTwo52;            // floor(v2 / q): qinv_up >= 1/q by less than 2^-49 relative
    const double rb = __fma_rn(-k, c.qd, v2 + kTwo52);                   // 2^52 + (v2 - k q), exact
    return (u64)__double_as_longlong(rb) & 0x000FFFFFFFFFFFFFull;
}
template <int STRIDE> __device__ __forceinline__ void fwd16_ds(double (&v)[16], const ulonglong2 *__restrict__ tp, const DsConst &c) {
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        const int half = 8 >> s;
#pragma unroll
        for (int g = 0; g < (1 << s); ++g) {
            const ulonglong2 tw = __ldg(tp + ((1 << s) - 1 + g) * STRIDE);
            const double wf = __longlong_as_double((long long)tw.y);
#pragma unroll
            for (int j = 0; j < half; ++j) {
                double &x = v[g * 2 * half + j], &y = v[g * 2 * half + j + half];
                const double t = ds_mul(y, tw.x, wf, c);
                y = x - t;
                x = x + t;
            }
        }
    }
}
template <int STRIDE> __device__ __forceinline__ void fwd16_ds8(double (&v)[16], const double *__restrict__ tp, const DsConst &c) {
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        const int half = 8 >> s;
#pragma unroll
        for (int g = 0; g < (1 << s); ++g) {
            const double wd = __ldg(tp + ((1 << s) - 1 + g) * STRIDE);
#pragma unroll
            for (int j = 0; j < half; ++j) {
                double &x = v[g * 2 * half + j], &y = v[g * 2 * half + j + half];
                const double t = ds_mul_w(y, wd, c);
                y = x - t;
                x = x + t;
            }
        }
    }
}
template <int STRIDE> __device__ __forceinline__ void inv16_ds8(double (&v)[16], const double *__restrict__ tp, const DsConst &c) {
#pragma unroll
    for (int s = 3; s >= 0; --s) {
        const int half = 8 >> s;
#pragma unroll
        for (int g = 0; g < (1 << s); ++g) {
            const double wd = __ldg(tp + ((1 << s) - 1 + g) * STRIDE);
#pragma unroll
            for (int j = 0; j < half; ++j) {
                double &x = v[g * 2 * half + j], &y = v[g * 2 * half + j + half];
                const double d = x - y;
                x = x + y;
                y = ds_mul_w(d, wd, c);
            }
        }
    }
    v[0] = ds_reduce(v[0], c);
}
// Gentleman-Sande round.  The sum path doubles per stage; only v[0] takes the sum at all four stages (16 x its
// inputs), v[1] ends below 4.2 q whatever came in, the others lower: the caller reduces v[0] after each round, so
// every round starts from values below 4.2 q and stays below 68 q.
template <int STRIDE> __device__ __forceinline__ void inv16_ds(double (&v)[16], const ulonglong2 *__restrict__ tp, const DsConst &c) {
#pragma unroll
    for (int s = 3; s >= 0; --s) {
        const int half = 8 >> s;
#pragma unroll
        for (int g = 0; g < (1 << s); ++g) {
            const ulonglong2 tw = __ldg(tp + ((1 << s) - 1 + g) * STRIDE);
            const double wf = __longlong_as_double((long long)tw.y);
#pragma unroll
            for (int j = 0; j < half; ++j) {
                double &x = v[g * 2 * half + j], &y = v[g * 2 * half + j + half];
                const double d = x - y;
                x = x + y;
                y = ds_mul(d, tw.x, wf, c);
            }
        }
    }
    v[0] = ds_reduce(v[0], c);
}

// ---- forward, column pass: stages 1..8 ----
template <int MINB>
__global__ void __launch_bounds__(256, MINB) ntt16v2_fwd_cols(const u64 *__restrict__ src, LimbAddr16 sa, u64 *__restrict__ dst, LimbAddr16 da,
                                                        const __grid_constant__ LimbMap map, const PrimeConst *__restrict__ pc, Ntt16Tables tb) {
    __shared__ u64 sm[4096];
    const int li = blockIdx.y, pi = map.prime[li % map.n];
    const PrimeConst m = pc[pi];
    const ulonglong2 *tab = tb.fwd + (size_t)pi * Ntt16Layout::kEntries;
    const int tid = threadIdx.x, lane = tid & 15, sub = tid >> 4;
    const u64 *p = src + sa.off(li, map.n) + blockIdx.x * 16 + lane;
    u64 *o = dst + da.off(li, map.n) + blockIdx.x * 16 + lane;
    if (m.small) {
        const DsConst c = ds_const(m);
        double v[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = ds_load(p[(e * 16 + sub) * 256]);
        fwd16_ds<1>(v, tab + Ntt16Layout::colsA(0), c);
        double *smd = reinterpret_cast<double *>(sm);
#pragma unroll
        for (int e = 0; e < 16; ++e) smd[(e * 16 + sub) * 16 + lane] = v[e];
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = smd[(sub * 16 + e) * 16 + lane];
        fwd16_ds<1>(v, tab + Ntt16Layout::colsB(sub, 0), c);
        double *od = reinterpret_cast<double *>(o);
#pragma unroll
        for (int e = 0; e < 16; ++e) od[(sub * 16 + e) * 256] = v[e];
    } else {
        u64 v[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = p[(e * 16 + sub) * 256];
        fwd16_int<1>(v, tab + Ntt16Layout::colsA(0), m.q);
#pragma unroll
        for (int e = 0; e < 16; ++e) sm[(e * 16 + sub) * 16 + lane] = v[e];
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = sm[(sub * 16 + e) * 16 + lane];
        fwd16_int<1>(v, tab + Ntt16Layout::colsB(sub, 0), m.q);
#pragma unroll
        for (int e = 0; e < 16; ++e) o[(sub * 16 + e) * 256] = v[e];
    }
}

// ---- forward, row pass: stages 9..16; stores canonical residues ----
template <int MINB>
__global__ void __launch_bounds__(256, MINB) ntt16v2_fwd_rows(const u64 *__restrict__ src, LimbAddr16 sa, u64 *__restrict__ dst, LimbAddr16 da,
                                                        const __grid_constant__ LimbMap map, const PrimeConst *__restrict__ pc, Ntt16Tables tb) {
    __shared__ u64 sm[16 * kRowStride];
    const int li = blockIdx.y, pi = map.prime[li % map.n];
    const PrimeConst m = pc[pi];
    const ulonglong2 *tab = tb.fwd + (size_t)pi * Ntt16Layout::kEntries;
    const int tid = threadIdx.x, clo = tid & 15, rl = tid >> 4;
    const int row = blockIdx.x * 16 + rl;
    const u64 *p = src + sa.off(li, map.n) + (size_t)row * 256 + clo;
    u64 *o = dst + da.off(li, map.n) + (size_t)row * 256 + clo;
    u64 *smr = sm + rl * kRowStride;
    if (m.small) {
        const DsConst c = ds_const(m);
        const double *pd = reinterpret_cast<const double *>(p);
        double *smd = reinterpret_cast<double *>(smr);
        double v[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = pd[e * 16];
        fwd16_ds<1>(v, tab + Ntt16Layout::rowsA(row, 0), c);
#pragma unroll
        for (int e = 0; e < 16; ++e) smd[e * 17 + clo] = v[e];
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = smd[clo * 17 + e];
        fwd16_ds8<16>(v, tb.fwdB8 + (size_t)pi * kRowsB8 + (row * 15) * 16 + clo, c);
        const double shift = 16.0 * c.qd, qinv_up = c.qinv * (1.0 + 0x1p-50);
#pragma unroll
        for (int e = 0; e < 16; ++e) smr[clo * 17 + e] = ds_store(v[e], c, shift, qinv_up); // the words this thread read itself
    } else {
        const u64 q = m.q, q2 = q << 1;
        u64 v[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = p[e * 16];
        fwd16_int<1>(v, tab + Ntt16Layout::rowsA(row, 0), q);
#pragma unroll
        for (int e = 0; e < 16; ++e) smr[e * 17 + clo] = v[e];
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = smr[clo * 17 + e];
        fwd16_int<16>(v, tab + Ntt16Layout::rowsB(row, 0, clo), q);
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            u64 x = v[e];
            x = x >= q2 ? x - q2 : x;
            smr[clo * 17 + e] = x >= q ? x - q : x;
        }
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 16; ++e) o[e * 16] = smr[e * 17 + clo];
}

// ---- inverse, row pass: undoes stages 16..9 ----
template <int MINB>
__global__ void __launch_bounds__(256, MINB) ntt16v2_inv_rows(const u64 *__restrict__ src, LimbAddr16 sa, u64 *__restrict__ dst, LimbAddr16 da,
                                                        const __grid_constant__ LimbMap map, const PrimeConst *__restrict__ pc, Ntt16Tables tb) {
    __shared__ u64 sm[16 * kRowStride];
    const int li = blockIdx.y, pi = map.prime[li % map.n];
    const PrimeConst m = pc[pi];
    const ulonglong2 *tab = tb.inv + (size_t)pi * Ntt16Layout::kEntries;
    const int tid = threadIdx.x, clo = tid & 15, rl = tid >> 4;
    const int row = blockIdx.x * 16 + rl;
    const u64 *p = src + sa.off(li, map.n) + (size_t)row * 256 + clo;
    u64 *o = dst + da.off(li, map.n) + (size_t)row * 256 + clo;
    u64 *smr = sm + rl * kRowStride;
#pragma unroll
    for (int e = 0; e < 16; ++e) smr[e * 17 + clo] = p[e * 16];
    __syncthreads();
    if (m.small) {
        const DsConst c = ds_const(m);
        double *smd = reinterpret_cast<double *>(smr);
        double v[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = ds_load(smr[clo * 17 + e]);
        inv16_ds8<16>(v, tb.invB8 + (size_t)pi * kRowsB8 + (row * 15) * 16 + clo, c);
#pragma unroll
        for (int e = 0; e < 16; ++e) smd[clo * 17 + e] = v[e]; // the words this thread read itself
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = smd[e * 17 + clo];
        inv16_ds<1>(v, tab + Ntt16Layout::rowsA(row, 0), c);
        double *od = reinterpret_cast<double *>(o);
#pragma unroll
        for (int e = 0; e < 16; ++e) od[e * 16] = v[e];
    } else {
        u64 v[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = smr[clo * 17 + e];
        inv16_int<16>(v, tab + Ntt16Layout::rowsB(row, 0, clo), m.q);
#pragma unroll
        for (int e = 0; e < 16; ++e) smr[clo * 17 + e] = v[e];
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = smr[e * 17 + clo];
        inv16_int<1>(v, tab + Ntt16Layout::rowsA(row, 0), m.q);
#pragma unroll
        for (int e = 0; e < 16; ++e) o[e * 16] = v[e];
    }
}

// ---- inverse, column pass: undoes stages 8..1, scales by N^-1, stores canonical residues ----
template <int MINB>
__global__ void __launch_bounds__(256, MINB) ntt16v2_inv_cols(const u64 *__restrict__ src, LimbAddr16 sa, u64 *__restrict__ dst, LimbAddr16 da,
                                                        const __grid_constant__ LimbMap map, const PrimeConst *__restrict__ pc, Ntt16Tables tb,
                                                        const __grid_constant__ Ntt16Scale sc) {
    __shared__ u64 sm[4096];
    const int li = blockIdx.y, pos = li % map.n, pi = map.prime[pos];
    const PrimeConst m = pc[pi];
    const ulonglong2 *tab = tb.inv + (size_t)pi * Ntt16Layout::kEntries;
    const int tid = threadIdx.x, lane = tid & 15, sub = tid >> 4;
    const u64 *p = src + sa.off(li, map.n) + blockIdx.x * 16 + lane;
    u64 *o = dst + da.off(li, map.n) + blockIdx.x * 16 + lane;
    if (m.small) {
        const DsConst c = ds_const(m);
        const double *pd = reinterpret_cast<const double *>(p);
        double *smd = reinterpret_cast<double *>(sm);
        double v[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = pd[(sub * 16 + e) * 256];
        inv16_ds<1>(v, tab + Ntt16Layout::colsB(sub, 0), c);
#pragma unroll
        for (int e = 0; e < 16; ++e) smd[(sub * 16 + e) * 16 + lane] = v[e];
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = smd[(e * 16 + sub) * 16 + lane];
        inv16_ds<1>(v, tab + Ntt16Layout::colsA(0), c);
        const double qinv_up = c.qinv * (1.0 + 0x1p-50);
        const u64 sw = sc.on ? sc.w[pos] : ds_twiddle_word(m.n_inv);
        const double sf = sc.on ? __longlong_as_double((long long)sc.comp[pos]) : m.n_inv_f;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const double t = ds_mul(v[e], sw, sf, c); // x * N^-1 (or x * scale) in (-0.52 q, 0.52 q)
            o[(e * 16 + sub) * 256] = ds_store(t, c, c.qd, qinv_up);
        }
    } else {
        u64 v[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = p[(sub * 16 + e) * 256];
        inv16_int<1>(v, tab + Ntt16Layout::colsB(sub, 0), m.q);
#pragma unroll
        for (int e = 0; e < 16; ++e) sm[(sub * 16 + e) * 16 + lane] = v[e];
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = sm[(e * 16 + sub) * 16 + lane];
        inv16_int<1>(v, tab + Ntt16Layout::colsA(0), m.q);
#pragma unroll
        const u64 sw = sc.on ? sc.w[pos] : m.n_inv, ss = sc.on ? sc.comp[pos] : m.n_inv_sh;
#pragma unroll
        for (int e = 0; e < 16; ++e) o[(e * 16 + sub) * 256] = mul_shoup(v[e], sw, ss, m.q);
    }
}

// Launch a batched transform of `count` limb instances of 2^16 coefficients.  src == dst gives an in-place transform;
// with distinct buffers `dst` also serves as the intermediate between the two passes.  MINB = CTAs per SM the kernels
// are compiled for (register budget 65536 / (256 * MINB)); four measured fastest with the FP64 butterflies.
template <int MINB = 4>
inline cudaError_t launch_ntt16(cudaStream_t st, const u64 *src, size_t src_outer, u64 *dst, size_t dst_outer, int count, const LimbMap &map,
                                const PrimeConst *pc, const Ntt16Tables &tb, bool inverse, const Ntt16Scale *scale = nullptr) {
    if (count == 0) return cudaSuccess;
    LimbAddr16 sa{src_outer}, da{dst_outer};
    dim3 grid(16, count);
    if (!inverse) {
        ntt16v2_fwd_cols<MINB><<<grid, 256, 0, st>>>(src, sa, dst, da, map, pc, tb);
        ntt16v2_fwd_rows<MINB><<<grid, 256, 0, st>>>(dst, da, dst, da, map, pc, tb);
    } else {
        ntt16v2_inv_rows<MINB><<<grid, 256, 0, st>>>(src, sa, dst, da, map, pc, tb);
        Ntt16Scale none{};
        ntt16v2_inv_cols<MINB><<<grid, 256, 0, st>>>(dst, da, dst, da, map, pc, tb, scale ? *scale : none);
    }
    return cudaGetLastError();
}

} // namespace hb
