// CPU ORACLE -- TEST INFRASTRUCTURE ONLY.  PARITY UNPINNED (see below).
//
// This header is a plain, scalar C++ restatement of the RNS-CKKS arithmetic that
// the reference obtains from the closed HEaaN library through the calls declared
// in ciphertext/external/include/HEaaN/{HomEvaluator,EnDecoder,Encryptor,
// Decryptor,KeyGenerator}.hpp.  The reference ships only those headers; the
// library binary is not available, and the reference holds no golden vectors,
// no known-answer tests and never seeds its randomness.  The residue-level
// behaviour is therefore defined by the specification written in the comments
// of this file ("parity unpinned" against HEaaN itself); what pins it is
//   * brute-force identities at tiny sizes (schoolbook negacyclic product,
//     big-integer CRT, direct evaluation of the canonical embedding),
//   * the ChaCha20 block-function known-answer vector of RFC 8439 section 2.3.2,
//   * decrypt-and-compare against float64 matmul with the tolerance the reference
//     uses (2^-14, ciphertext/test/HELLMTestBase.hpp:34).
//
// Nothing in the shipped library may include, link or call this file.  It is used
// by tests/, by the smoke check and by the cpu-baseline leg of the benchmark.
//
// Specification summary (every quantity is exact integer arithmetic unless noted):
//   ring        R_q = Z_q[X]/(X^N+1), N = 2^log_n, slots = N/2
//   moduli      index 0..L: q_0 (q0_bits) then scaling primes q_1..q_L (< 2^q_bits),
//               index L+1..L+K: special primes p_0..p_{K-1}; all == 1 (mod 2N)
//   NTT form    a_hat[i] = a(psi^(2*bitrev(i)+1)), psi = x^((q-1)/2N) for the smallest
//               x >= 2 that makes psi^N == -1
//   scale       Delta_L = 2^q_bits, Delta_{l-1} = Delta_l^2 / q_l  (IEEE double)
//   ciphertext  (b, a) with b + a*s = m + e, both polys in NTT form, limb-major
//   key switch  hybrid; limb i belongs to digit (i+1)/alpha, alpha = ceil((L+2)/dnum), so the
//               digit that holds the wide q_0 has one limb fewer and every digit product
//               stays below P = prod p_j (a digit wider than P costs ~N*Q_digit/P of noise);
//               approximate fast base conversion without correction term
//   rotation    decompose-then-permute (see Evaluator::keyswitch)
#pragma once
#include <algorithm>
#include <array>
#include <cmath>
#include <complex>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace orc {

using u32 = uint32_t;
using u64 = uint64_t;
using i64 = int64_t;
using u128 = unsigned __int128;
using i128 = __int128;
using cplx = std::complex<double>;

// ---------------------------------------------------------------------------
// Modular arithmetic for one word-sized prime q < 2^62.
// ---------------------------------------------------------------------------
struct Mod {
    u64 q = 0;
    u64 mu_hi = 0, mu_lo = 0; // floor(2^128 / q) as two words

    void init(u64 q_) {
        q = q_;
        u128 two64 = (u128)1 << 64;
        mu_hi = (u64)(two64 / q);
        u128 r = two64 % q;
        mu_lo = (u64)((r << 64) / q);
    }
    // z mod q for any 128-bit z (Barrett, quotient estimate low by at most 3)
    u64 red128(u128 z) const {
        u64 z1 = (u64)(z >> 64), z0 = (u64)z;
        u64 qh = z1 * mu_hi + (u64)(((u128)z1 * mu_lo) >> 64) + (u64)(((u128)z0 * mu_hi) >> 64);
        u64 r = z0 - qh * q;
        while (r >= q) r -= q;
        return r;
    }
    u64 red(u64 x) const { return x % q; }
    u64 mul(u64 a, u64 b) const { return red128((u128)a * b); }
    u64 add(u64 a, u64 b) const { u64 s = a + b; return s >= q ? s - q : s; }
    u64 sub(u64 a, u64 b) const { return a >= b ? a - b : a + q - b; }
    u64 neg(u64 a) const { return a ? q - a : 0; }
    u64 pow(u64 a, u64 e) const {
        u64 r = 1; a %= q;
        while (e) { if (e & 1) r = mul(r, a); a = mul(a, a); e >>= 1; }
        return r;
    }
    u64 inv(u64 a) const { return pow(a, q - 2); }
    u64 from_i64(i64 v) const {
        if (v >= 0) return (u64)v % q;
        u64 r = (u64)(-(v + 1)) % q; // -(v+1) avoids overflow at INT64_MIN
        return q - 1 - r;
    }
    u64 shoup(u64 w) const { return (u64)(((u128)w << 64) / q); }
    static u64 mul_shoup(u64 x, u64 w, u64 wsh, u64 q) {
        u64 hi = (u64)(((u128)x * wsh) >> 64);
        u64 r = x * w - hi * q;
        return r >= q ? r - q : r;
    }
};

inline bool is_prime_u64(u64 n) {
    if (n < 2) return false;
    for (u64 p : {2ull, 3ull, 5ull, 7ull, 11ull, 13ull, 17ull, 19ull, 23ull, 29ull, 31ull, 37ull}) {
        if (n % p == 0) return n == p;
    }
    u64 d = n - 1; int s = 0;
    while ((d & 1) == 0) { d >>= 1; ++s; }
    auto mulm = [&](u64 a, u64 b) { return (u64)(((u128)a * b) % n); };
    auto powm = [&](u64 a, u64 e) { u64 r = 1; while (e) { if (e & 1) r = mulm(r, a); a = mulm(a, a); e >>= 1; } return r; };
    for (u64 a : {2ull, 3ull, 5ull, 7ull, 11ull, 13ull, 17ull, 19ull, 23ull, 29ull, 31ull, 37ull}) {
        u64 x = powm(a, d);
        if (x == 1 || x == n - 1) continue;
        bool comp = true;
        for (int r = 1; r < s; ++r) { x = mulm(x, x); if (x == n - 1) { comp = false; break; } }
        if (comp) return false;
    }
    return true;
}

inline u32 bitrev(u32 x, int bits) {
    u32 r = 0;
    for (int i = 0; i < bits; ++i) { r = (r << 1) | (x & 1); x >>= 1; }
    return r;
}

// ---------------------------------------------------------------------------
// ChaCha20 block function (RFC 8439).  Stream addressing used by this library:
// key = the 256-bit seed, counter = block index, nonce = (domain, id_lo, id_hi).
// ---------------------------------------------------------------------------
struct ChaCha {
    u32 key[8];
    void set_seed(const u64 seed[4]) {
        for (int i = 0; i < 4; ++i) { key[2 * i] = (u32)seed[i]; key[2 * i + 1] = (u32)(seed[i] >> 32); }
    }
    static inline u32 rotl(u32 v, int c) { return (v << c) | (v >> (32 - c)); }
    static void core(const u32 in[16], u32 out[16]) {
        u32 x[16];
        for (int i = 0; i < 16; ++i) x[i] = in[i];
        auto qr = [&](int a, int b, int c, int d) {
            x[a] += x[b]; x[d] ^= x[a]; x[d] = rotl(x[d], 16);
            x[c] += x[d]; x[b] ^= x[c]; x[b] = rotl(x[b], 12);
            x[a] += x[b]; x[d] ^= x[a]; x[d] = rotl(x[d], 8);
            x[c] += x[d]; x[b] ^= x[c]; x[b] = rotl(x[b], 7);
        };
        for (int r = 0; r < 10; ++r) {
            qr(0, 4, 8, 12); qr(1, 5, 9, 13); qr(2, 6, 10, 14); qr(3, 7, 11, 15);
            qr(0, 5, 10, 15); qr(1, 6, 11, 12); qr(2, 7, 8, 13); qr(3, 4, 9, 14);
        }
        for (int i = 0; i < 16; ++i) out[i] = x[i] + in[i];
    }
    void block(u32 domain, u64 id, u32 counter, u32 out[16]) const {
        u32 st[16] = {0x61707865u, 0x3320646eu, 0x79622d32u, 0x6b206574u};
        for (int i = 0; i < 8; ++i) st[4 + i] = key[i];
        st[12] = counter; st[13] = domain; st[14] = (u32)id; st[15] = (u32)(id >> 32);
        core(st, out);
    }
    // t-th 64-bit word of stream (domain, id)
    u64 word64(u32 domain, u64 id, u64 t) const {
        u32 o[16]; block(domain, id, (u32)(t >> 3), o);
        int k = (int)(t & 7);
        return (u64)o[2 * k] | ((u64)o[2 * k + 1] << 32);
    }
};

enum : u32 { DOM_SK = 1, DOM_ENC_A = 2, DOM_ENC_E = 3, DOM_KEY_A = 4, DOM_KEY_E = 5 };

struct Params {
    int log_n = 16, max_level = 12, dnum = 4, num_special = 3;
    int q0_bits = 60, q_bits = 42, p_bits = 60, hamming_weight = 192;
    double sigma = 3.2;
    u64 seed[4] = {1, 2, 3, 4};
};

// ---------------------------------------------------------------------------
// Context: primes, NTT tables, scales, encoder tables, base-conversion constants.
// ---------------------------------------------------------------------------
struct Context {
    Params prm;
    int logN, N, slots, L, K, alpha, nprimes;
    std::vector<Mod> mod;                       // [L+1+K]
    std::vector<std::vector<u64>> psi, psi_sh;  // psi^bitrev(k) and Shoup companion
    std::vector<std::vector<u64>> ipsi, ipsi_sh;
    std::vector<u64> n_inv, n_inv_sh, imag_unit; // N^-1 mod q ; psi^(N/2)
    std::vector<double> scale;                  // Delta_l
    std::vector<u64> rot_group;                 // 5^j mod 2N
    std::vector<cplx> ksi;                      // exp(2 pi i k / 2N)
    std::vector<u64> cdt;                       // Gaussian cumulative table (63-bit)
    ChaCha rng;
    std::vector<i64> sk_coeff;                  // ternary secret, coefficient form
    std::vector<std::vector<u64>> sk_ntt;       // [nprimes][N]
    std::map<u64, std::vector<u32>> perm_cache; // galois element -> NTT-domain gather

    explicit Context(const Params &p) : prm(p) {
        logN = p.log_n; N = 1 << logN; slots = N / 2; L = p.max_level; K = p.num_special;
        alpha = (L + 2 + p.dnum - 1) / p.dnum; nprimes = L + 1 + K;
        {   // every digit product must stay below P
            int pbits = K * p.p_bits;
            int d0 = p.q0_bits + std::max(0, std::min(alpha - 2, L)) * p.q_bits, dk = alpha * p.q_bits;
            if (d0 > pbits || (L + 1 > alpha - 1 && dk > pbits)) throw std::invalid_argument("special modulus narrower than a key-switch digit");
        }
        if (p.hamming_weight > N) throw std::invalid_argument("hamming weight > N");
        rng.set_seed(p.seed);
        choose_primes();
        build_ntt_tables();
        build_encoder_tables();
        build_cdt();
    }

    // Prime-selection rule.  Candidates of a size class are 2^bits - t*2N + 1, t = 1,2,...
    //   q_0   = first prime of the q0_bits class;
    //   p_j   = next K primes of the p_bits class (skipping q_0);
    //   q_l   (l = L..1) = the unused prime of the q_bits class nearest to
    //           Delta_l^2 / 2^q_bits (ties to the larger), Delta_{l-1} = Delta_l^2 / q_l.
    void choose_primes() {
        const u64 twoN = (u64)2 * N;
        auto cands = [&](int bits, int count) {
            std::vector<u64> v; u64 c = ((u64)1 << bits) + 1;
            while ((int)v.size() < count) { c -= twoN; if (is_prime_u64(c)) v.push_back(c); }
            return v;
        };
        std::vector<u64> primes(nprimes);
        primes[0] = cands(prm.q0_bits, 1)[0];
        {
            auto pc = cands(prm.p_bits, K + 1); int t = 0;
            for (int j = 0; j < K; ++j) { if (pc[t] == primes[0]) ++t; primes[L + 1 + j] = pc[t++]; }
        }
        scale.assign(L + 1, 0.0);
        scale[L] = std::ldexp(1.0, prm.q_bits);
        auto sc = cands(prm.q_bits, 4 * L + 4);
        std::vector<char> used(sc.size(), 0);
        for (int l = L; l >= 1; --l) {
            double target = scale[l] * scale[l] / std::ldexp(1.0, prm.q_bits);
            int best = -1; double bd = 0;
            for (size_t i = 0; i < sc.size(); ++i) {
                if (used[i] || sc[i] == primes[0]) continue;
                double d = std::fabs((double)sc[i] - target);
                if (best < 0 || d < bd) { best = (int)i; bd = d; }
            }
            used[best] = 1; primes[l] = sc[best];
            scale[l - 1] = scale[l] * scale[l] / (double)primes[l];
        }
        mod.resize(nprimes);
        for (int i = 0; i < nprimes; ++i) mod[i].init(primes[i]);
    }

    void build_ntt_tables() {
        psi.resize(nprimes); psi_sh.resize(nprimes); ipsi.resize(nprimes); ipsi_sh.resize(nprimes);
        n_inv.resize(nprimes); n_inv_sh.resize(nprimes); imag_unit.resize(nprimes);
        for (int pi = 0; pi < nprimes; ++pi) {
            const Mod &m = mod[pi];
            u64 root = 0;
            for (u64 x = 2;; ++x) {
                u64 c = m.pow(x, (m.q - 1) / ((u64)2 * N));
                if (m.pow(c, N) == m.q - 1) { root = c; break; }
            }
            u64 iroot = m.inv(root);
            std::vector<u64> pw(N), ipw(N);
            pw[0] = ipw[0] = 1;
            for (int k = 1; k < N; ++k) { pw[k] = m.mul(pw[k - 1], root); ipw[k] = m.mul(ipw[k - 1], iroot); }
            psi[pi].resize(N); psi_sh[pi].resize(N); ipsi[pi].resize(N); ipsi_sh[pi].resize(N);
            for (int k = 0; k < N; ++k) {
                u32 r = bitrev((u32)k, logN);
                psi[pi][k] = pw[r]; psi_sh[pi][k] = m.shoup(pw[r]);
                ipsi[pi][k] = ipw[r]; ipsi_sh[pi][k] = m.shoup(ipw[r]);
            }
            n_inv[pi] = m.inv((u64)N); n_inv_sh[pi] = m.shoup(n_inv[pi]);
            imag_unit[pi] = pw[N / 2];
        }
    }

    void build_encoder_tables() {
        const u64 M = (u64)2 * N;
        rot_group.resize(slots);
        u64 g = 1;
        for (int j = 0; j < slots; ++j) { rot_group[j] = g; g = (g * 5) % M; }
        ksi.resize(M + 1);
        const double pi = 3.14159265358979323846264338327950288;
        for (u64 k = 0; k <= M; ++k) {
            double ang = 2.0 * pi * (double)k / (double)M;
            ksi[k] = cplx(std::cos(ang), std::sin(ang));
        }
    }

    // Discrete Gaussian by cumulative table: magnitudes 0..J, J = ceil(13 sigma).
    // cdt[k] = floor(2^63 * P(|x| <= k)); a 63-bit uniform u has magnitude #{k : cdt[k] <= u}.
    void build_cdt() {
        int J = (int)std::ceil(13.0 * prm.sigma);
        std::vector<double> rho(J + 1);
        double S = 1.0;
        for (int j = 0; j <= J; ++j) rho[j] = std::exp(-(double)j * (double)j / (2.0 * prm.sigma * prm.sigma));
        for (int j = 1; j <= J; ++j) S += 2.0 * rho[j];
        cdt.resize(J);
        double cum = 0.0;
        for (int k = 0; k < J; ++k) {
            cum += (k == 0 ? rho[0] : 2.0 * rho[k]) / S;
            double v = std::floor(std::ldexp(cum, 63));
            cdt[k] = v >= 9223372036854775808.0 ? ((u64)1 << 63) : (u64)v;
        }
    }

    int digit_of(int limb) const { return (limb + 1) / alpha; }
    int digit_lo(int dg) const { return std::max(0, dg * alpha - 1); }
    int digit_hi(int dg, int n) const { return std::min((dg + 1) * alpha - 1, n); } // exclusive, n = level+1
    int num_digits(int level) const { return digit_of(level) + 1; }
    u64 galois_for_rotation(i64 left_steps) const {
        i64 r = left_steps % slots; if (r < 0) r += slots;
        return rot_group[(size_t)r];
    }
    u64 galois_conj() const { return (u64)2 * N - 1; }

    // gather table for the automorphism X -> X^g applied to an NTT-form limb:
    //   out[i] = in[perm[i]],  (2*bitrev(perm[i])+1) == g*(2*bitrev(i)+1)  (mod 2N)
    const std::vector<u32> &ntt_perm(u64 g) {
        auto it = perm_cache.find(g);
        if (it != perm_cache.end()) return it->second;
        std::vector<u32> p(N);
        const u64 mask = (u64)2 * N - 1;
        for (int i = 0; i < N; ++i) {
            u64 e = (u64)2 * bitrev((u32)i, logN) + 1;
            u64 ej = (g * e) & mask;
            p[i] = bitrev((u32)((ej - 1) >> 1), logN);
        }
        return perm_cache.emplace(g, std::move(p)).first->second;
    }

    // ----- NTT (Cooley-Tukey forward, Gentleman-Sande inverse, fully reduced) -----
    void ntt(u64 *a, int pi) const {
        const Mod &m = mod[pi]; const u64 q = m.q;
        const u64 *w = psi[pi].data(), *ws = psi_sh[pi].data();
        int t = N;
        for (int mm = 1; mm < N; mm <<= 1) {
            t >>= 1;
            for (int i = 0; i < mm; ++i) {
                u64 W = w[mm + i], Ws = ws[mm + i];
                u64 *x = a + 2 * i * t, *y = x + t;
                for (int j = 0; j < t; ++j) {
                    u64 U = x[j], V = Mod::mul_shoup(y[j], W, Ws, q);
                    u64 s = U + V; x[j] = s >= q ? s - q : s;
                    y[j] = U >= V ? U - V : U + q - V;
                }
            }
        }
    }
    void intt(u64 *a, int pi) const {
        const Mod &m = mod[pi]; const u64 q = m.q;
        const u64 *w = ipsi[pi].data(), *ws = ipsi_sh[pi].data();
        int t = 1;
        for (int mm = N >> 1; mm >= 1; mm >>= 1) {
            for (int i = 0; i < mm; ++i) {
                u64 W = w[mm + i], Ws = ws[mm + i];
                u64 *x = a + 2 * i * t, *y = x + t;
                for (int j = 0; j < t; ++j) {
                    u64 U = x[j], V = y[j];
                    u64 s = U + V; x[j] = s >= q ? s - q : s;
                    u64 d = U >= V ? U - V : U + q - V;
                    y[j] = Mod::mul_shoup(d, W, Ws, q);
                }
            }
            t <<= 1;
        }
        for (int j = 0; j < N; ++j) a[j] = Mod::mul_shoup(a[j], n_inv[pi], n_inv_sh[pi], q);
    }

    // ----- canonical embedding (special FFT over the orbit of 5) -----
    static void bitrev_array(std::vector<cplx> &v) {
        size_t n = v.size();
        for (size_t i = 1, j = 0; i < n; ++i) {
            size_t bit = n >> 1;
            for (; j >= bit; bit >>= 1) j -= bit;
            j += bit;
            if (i < j) std::swap(v[i], v[j]);
        }
    }
    static inline cplx cmul(cplx a, cplx b) {
        return cplx(a.real() * b.real() - a.imag() * b.imag(), a.real() * b.imag() + a.imag() * b.real());
    }
    void fft_special(std::vector<cplx> &v) const { // coefficients-side -> slots
        const size_t n = v.size(); const u64 M = (u64)2 * N;
        bitrev_array(v);
        for (size_t len = 2; len <= n; len <<= 1) {
            size_t lenh = len >> 1, lenq = len << 2; u64 gap = M / lenq;
            for (size_t i = 0; i < n; i += len)
                for (size_t j = 0; j < lenh; ++j) {
                    u64 idx = (rot_group[j] % lenq) * gap;
                    cplx u = v[i + j], w = cmul(v[i + j + lenh], ksi[idx]);
                    v[i + j] = cplx(u.real() + w.real(), u.imag() + w.imag());
                    v[i + j + lenh] = cplx(u.real() - w.real(), u.imag() - w.imag());
                }
        }
    }
    void fft_special_inv(std::vector<cplx> &v) const { // slots -> coefficients-side
        const size_t n = v.size(); const u64 M = (u64)2 * N;
        for (size_t len = n; len >= 2; len >>= 1) {
            size_t lenh = len >> 1, lenq = len << 2; u64 gap = M / lenq;
            for (size_t i = 0; i < n; i += len)
                for (size_t j = 0; j < lenh; ++j) {
                    u64 idx = (lenq - (rot_group[j] % lenq)) * gap;
                    cplx u(v[i + j].real() + v[i + j + lenh].real(), v[i + j].imag() + v[i + j + lenh].imag());
                    cplx d(v[i + j].real() - v[i + j + lenh].real(), v[i + j].imag() - v[i + j + lenh].imag());
                    v[i + j] = u; v[i + j + lenh] = cmul(d, ksi[idx]);
                }
        }
        bitrev_array(v);
        const double inv = 1.0 / (double)n;
        for (auto &x : v) x = cplx(x.real() * inv, x.imag() * inv);
    }

    // ----- samplers -----
    void sample_uniform_limb(u32 domain, u64 id, int pi, u64 *out) const {
        const Mod &m = mod[pi];
        for (int c = 0; c < N; c += 4) {
            u32 o[16];
            u64 s = (u64)pi * N + c;
            rng.block(domain, id, (u32)(s >> 2), o);
            for (int k = 0; k < 4; ++k) {
                u64 lo = (u64)o[4 * k] | ((u64)o[4 * k + 1] << 32);
                u64 hi = (u64)o[4 * k + 2] | ((u64)o[4 * k + 3] << 32);
                out[c + k] = m.red128(((u128)hi << 64) | lo);
            }
        }
    }
    void sample_gauss(u32 domain, u64 id, std::vector<i64> &out) const {
        out.resize(N);
        for (int c = 0; c < N; ++c) {
            u64 r = rng.word64(domain, id, (u64)c);
            u64 u = r >> 1; i64 mag = 0;
            for (u64 t : cdt) mag += (t <= u);
            out[c] = (r & 1) ? -mag : mag;
        }
    }
    void gen_secret() {
        sk_coeff.assign(N, 0);
        int cnt = 0; u64 t = 0;
        while (cnt < prm.hamming_weight) {
            u64 r = rng.word64(DOM_SK, 0, t++);
            size_t pos = (size_t)(r & (u64)(N - 1));
            if (sk_coeff[pos] != 0) continue;
            sk_coeff[pos] = (r >> 63) ? -1 : 1; ++cnt;
        }
        sk_ntt.assign(nprimes, std::vector<u64>(N));
#pragma omp parallel for
        for (int pi = 0; pi < nprimes; ++pi) {
            for (int c = 0; c < N; ++c) sk_ntt[pi][c] = mod[pi].from_i64(sk_coeff[c]);
            ntt(sk_ntt[pi].data(), pi);
        }
    }
    int prime_index_ext(int level, int j) const { return j <= level ? j : L + 1 + (j - level - 1); }
};

// ---------------------------------------------------------------------------
// Data objects.  A "batch" holds several independent ciphertexts of equal level.
// ---------------------------------------------------------------------------
struct Ct {
    int level = -1, np = 2, spow = 1, batch = 1, N = 0;
    std::vector<u64> d; // [batch][np][level+1][N]
    Ct() {}
    Ct(int N_, int level_, int np_ = 2, int batch_ = 1, int spow_ = 1, bool meta_only = false)
        : level(level_), np(np_), spow(spow_), batch(batch_), N(N_), d(meta_only ? 0 : (size_t)batch_ * np_ * (level_ + 1) * N_, 0) {}
    u64 *limb(int b, int p, int l) { return d.data() + (((size_t)b * np + p) * (level + 1) + l) * N; }
    const u64 *limb(int b, int p, int l) const { return d.data() + (((size_t)b * np + p) * (level + 1) + l) * N; }
};
struct Pt {
    int level = -1, spow = 1, N = 0;
    bool ext = false;   // K more limbs follow, modulo the special primes (operand of assemble_rot)
    std::vector<u64> d; // [level+1 (+K)][N] NTT form
    u64 *limb(int l) { return d.data() + (size_t)l * N; }
    const u64 *limb(int l) const { return d.data() + (size_t)l * N; }
};
struct Evk { // [digit][2][L+1+K][N], NTT form
    int nd = 0, nprimes = 0, N = 0;
    std::vector<u64> d;
    const u64 *limb(int dig, int p, int pi) const { return d.data() + (((size_t)dig * 2 + p) * nprimes + pi) * N; }
    u64 *limb(int dig, int p, int pi) { return d.data() + (((size_t)dig * 2 + p) * nprimes + pi) * N; }
};

// ---------------------------------------------------------------------------
// Evaluator: encode / encrypt / decrypt / key generation / homomorphic primitives.
// Semantics follow the doc comments of the HEaaN headers cited per function.
// ---------------------------------------------------------------------------
struct Evaluator {
    Context &cx;
    Evk mult_key;                 // key id 0 (s^2 -> s)
    std::map<u64, Evk> gal_keys;  // galois element -> key
    explicit Evaluator(Context &c) : cx(c) {}

    // Dry mode: every primitive keeps the level / shape bookkeeping but skips the arithmetic, and
    // counts itself in `stats`.  Used to obtain exact operation counts of a full-size schedule
    // (the cpu-baseline leg multiplies them by sampled per-operation times).
    bool dry = false;
    std::map<std::pair<std::string, int>, long> stats;
    bool count(const char *op, int level, int batch = 1) { if (dry) stats[{op, level}] += batch; return dry; }
    Ct meta(int level, int np, int batch, int spow) const { return Ct(cx.N, level, np, batch, spow, true); }

    // EnDecoder::encode (HEaaN/EnDecoder.hpp:51): slots -> plaintext at `level`, scale Delta_level
    Pt encode(const cplx *z, size_t n, int level) const {
        if ((int)n > cx.slots) throw std::invalid_argument("encode: too many slots");
        if (level < 0 || level > cx.L) throw std::invalid_argument("encode: bad level");
        if (dry) { ++const_cast<Evaluator *>(this)->stats[{"encode", level}]; Pt e; e.level = level; e.N = cx.N; return e; }
        std::vector<cplx> v(cx.slots, cplx(0, 0));
        for (size_t i = 0; i < n; ++i) v[i] = z[i];
        cx.fft_special_inv(v);
        const double sc = cx.scale[level];
        std::vector<i64> coef(cx.N);
        for (int i = 0; i < cx.slots; ++i) {
            coef[i] = (i64)std::rint(v[i].real() * sc);
            coef[i + cx.slots] = (i64)std::rint(v[i].imag() * sc);
        }
        Pt pt; pt.level = level; pt.N = cx.N; pt.d.resize((size_t)(level + 1) * cx.N);
#pragma omp parallel for
        for (int l = 0; l <= level; ++l) {
            u64 *p = pt.limb(l);
            for (int c = 0; c < cx.N; ++c) p[c] = cx.mod[l].from_i64(coef[c]);
            cx.ntt(p, l);
        }
        return pt;
    }
    // The same plaintext with K further limbs modulo the special primes, so that it can multiply a key-switch
    // result that is still in the basis Q_level u P.  The first level+1 limbs are those of encode().
    Pt encode_ext(const cplx *z, size_t n, int level) const {
        if ((int)n > cx.slots) throw std::invalid_argument("encode: too many slots");
        if (level < 0 || level > cx.L) throw std::invalid_argument("encode: bad level");
        if (dry) { ++const_cast<Evaluator *>(this)->stats[{"encode", level}]; Pt e; e.level = level; e.N = cx.N; e.ext = true; return e; }
        std::vector<cplx> v(cx.slots, cplx(0, 0));
        for (size_t i = 0; i < n; ++i) v[i] = z[i];
        cx.fft_special_inv(v);
        const double sc = cx.scale[level];
        std::vector<i64> coef(cx.N);
        for (int i = 0; i < cx.slots; ++i) {
            coef[i] = (i64)std::rint(v[i].real() * sc);
            coef[i + cx.slots] = (i64)std::rint(v[i].imag() * sc);
        }
        const int ne = level + 1 + cx.K;
        Pt pt; pt.level = level; pt.N = cx.N; pt.ext = true; pt.d.resize((size_t)ne * cx.N);
#pragma omp parallel for
        for (int j = 0; j < ne; ++j) {
            const int pi = cx.prime_index_ext(level, j);
            u64 *p = pt.limb(j);
            for (int c = 0; c < cx.N; ++c) p[c] = cx.mod[pi].from_i64(coef[c]);
            cx.ntt(p, pi);
        }
        return pt;
    }
    // coefficient-form limbs 0 (and 1) -> slots.  Uses limb 0 alone at level 0 and the
    // two-limb CRT otherwise; the value is centred modulo the product.
    void decode_coeff(const u64 *c0, const u64 *c1, int level, int spow, cplx *out) const {
        const double sc = spow == 2 ? cx.scale[level] * cx.scale[level] : cx.scale[level];
        std::vector<double> val(cx.N);
        if (level == 0 || c1 == nullptr) {
            const u64 q = cx.mod[0].q;
            for (int c = 0; c < cx.N; ++c) {
                u64 r = c0[c];
                val[c] = r > q / 2 ? -(double)(q - r) : (double)r;
            }
        } else {
            const Mod &m1 = cx.mod[1]; const u64 q0 = cx.mod[0].q;
            const u64 q0inv = m1.inv(q0 % m1.q);
            const u128 Q = (u128)q0 * m1.q;
            for (int c = 0; c < cx.N; ++c) {
                u64 r0 = c0[c], r1 = c1[c];
                u64 t = m1.mul(m1.sub(r1, r0 % m1.q), q0inv);
                u128 x = (u128)r0 + (u128)q0 * t;
                val[c] = x > Q / 2 ? -(double)(i128)(Q - x) : (double)(i128)x;
            }
        }
        std::vector<cplx> v(cx.slots);
        for (int i = 0; i < cx.slots; ++i) v[i] = cplx(val[i] / sc, val[i + cx.slots] / sc);
        cx.fft_special(v);
        for (int i = 0; i < cx.slots; ++i) out[i] = v[i];
    }
    // EnDecoder::decode (HEaaN/EnDecoder.hpp:66)
    void decode(const Pt &pt, cplx *out) const {
        std::vector<u64> c0(pt.limb(0), pt.limb(0) + cx.N), c1;
        cx.intt(c0.data(), 0);
        if (pt.level >= 1) { c1.assign(pt.limb(1), pt.limb(1) + cx.N); cx.intt(c1.data(), 1); }
        decode_coeff(c0.data(), pt.level >= 1 ? c1.data() : nullptr, pt.level, pt.spow, out);
    }

    // Encryptor::encrypt(ptxt, sk, ctxt) (HEaaN/Encryptor.hpp:84), symmetric:
    //   a uniform (stream ENC_A, nonce), e Gaussian (stream ENC_E, nonce), b = -a*s + e + m
    Ct encrypt(const Pt &pt, u64 nonce) const {
        if (dry) { ++const_cast<Evaluator *>(this)->stats[{"encrypt", pt.level}]; return meta(pt.level, 2, 1, pt.spow); }
        Ct ct(cx.N, pt.level, 2, 1, pt.spow);
        std::vector<i64> e; cx.sample_gauss(DOM_ENC_E, nonce, e);
#pragma omp parallel for
        for (int l = 0; l <= pt.level; ++l) {
            const Mod &m = cx.mod[l];
            u64 *b = ct.limb(0, 0, l), *a = ct.limb(0, 1, l);
            cx.sample_uniform_limb(DOM_ENC_A, nonce, l, a);
            std::vector<u64> en(cx.N);
            for (int c = 0; c < cx.N; ++c) en[c] = m.from_i64(e[c]);
            cx.ntt(en.data(), l);
            const u64 *s = cx.sk_ntt[l].data(), *mp = pt.limb(l);
            for (int c = 0; c < cx.N; ++c) b[c] = m.add(m.sub(en[c], m.mul(a[c], s[c])), mp[c]);
        }
        return ct;
    }
    // Decryptor::decrypt (HEaaN/Decryptor.hpp:36): b + a*s (+ d2*s^2), then decode
    void decrypt(const Ct &ct, int b, cplx *out) const {
        int nl = ct.level >= 1 ? 2 : 1;
        std::vector<std::vector<u64>> c(nl, std::vector<u64>(cx.N));
        for (int l = 0; l < nl; ++l) {
            const Mod &m = cx.mod[l]; const u64 *s = cx.sk_ntt[l].data();
            for (int i = 0; i < cx.N; ++i) {
                u64 v = m.add(ct.limb(b, 0, l)[i], m.mul(ct.limb(b, 1, l)[i], s[i]));
                if (ct.np == 3) v = m.add(v, m.mul(ct.limb(b, 2, l)[i], m.mul(s[i], s[i])));
                c[l][i] = v;
            }
            cx.intt(c[l].data(), l);
        }
        decode_coeff(c[0].data(), nl == 2 ? c[1].data() : nullptr, ct.level, ct.spow, out);
    }

    // KeyGenerator (HEaaN/KeyGenerator.hpp:89,160-165): switching key from s' to s.
    //   digit b, prime i:  b_b[i] = -a_b[i]*s[i] + e_b[i] + [i in digit b] * (P mod q_i) * s'[i]
    //   a_b from stream (KEY_A, kid*64+b), e_b from stream (KEY_E, kid*64+b)
    Evk gen_switch_key(u64 kid, const std::vector<std::vector<u64>> &sprime_ntt) const {
        Evk k; k.nd = cx.num_digits(cx.L); k.nprimes = cx.nprimes; k.N = cx.N;
        k.d.resize((size_t)k.nd * 2 * cx.nprimes * cx.N);
        for (int dg = 0; dg < k.nd; ++dg) {
            std::vector<i64> e; cx.sample_gauss(DOM_KEY_E, kid * 64 + dg, e);
#pragma omp parallel for
            for (int pi = 0; pi < cx.nprimes; ++pi) {
                const Mod &m = cx.mod[pi];
                u64 *b = k.limb(dg, 0, pi), *a = k.limb(dg, 1, pi);
                cx.sample_uniform_limb(DOM_KEY_A, kid * 64 + dg, pi, a);
                std::vector<u64> en(cx.N);
                for (int c = 0; c < cx.N; ++c) en[c] = m.from_i64(e[c]);
                cx.ntt(en.data(), pi);
                bool in_digit = pi <= cx.L && cx.digit_of(pi) == dg;
                u64 pmod = 1;
                if (in_digit) for (int j = 0; j < cx.K; ++j) pmod = m.mul(pmod, cx.mod[cx.L + 1 + j].q % m.q);
                const u64 *s = cx.sk_ntt[pi].data();
                for (int c = 0; c < cx.N; ++c) {
                    u64 v = m.sub(en[c], m.mul(a[c], s[c]));
                    if (in_digit) v = m.add(v, m.mul(pmod, sprime_ntt[pi][c]));
                    b[c] = v;
                }
            }
        }
        return k;
    }
    void keygen() { // secret + multiplication key + conjugation key
        cx.gen_secret();
        std::vector<std::vector<u64>> s2(cx.nprimes, std::vector<u64>(cx.N));
        for (int pi = 0; pi < cx.nprimes; ++pi)
            for (int c = 0; c < cx.N; ++c) s2[pi][c] = cx.mod[pi].mul(cx.sk_ntt[pi][c], cx.sk_ntt[pi][c]);
        mult_key = gen_switch_key(0, s2);
        gen_galois_key(cx.galois_conj());
    }
    void gen_galois_key(u64 g) {
        if (dry || gal_keys.count(g)) return;
        const auto &perm = cx.ntt_perm(g);
        std::vector<std::vector<u64>> sp(cx.nprimes, std::vector<u64>(cx.N));
        for (int pi = 0; pi < cx.nprimes; ++pi)
            for (int c = 0; c < cx.N; ++c) sp[pi][c] = cx.sk_ntt[pi][perm[c]];
        gal_keys.emplace(g, gen_switch_key(g, sp));
    }
    void gen_rot_key(i64 left_steps) {
        u64 g = cx.galois_for_rotation(left_steps);
        if (g != 1) gen_galois_key(g);
    }

    // Fast base conversion of one coefficient column: in[] residues w.r.t. primes src[],
    // result modulo prime index dst:  sum_i [x_i * (B/b_i)^-1]_{b_i} * (B/b_i) mod dst.
    struct BConv {
        std::vector<int> src; std::vector<u64> hat_inv, hat_inv_sh; // per source
        std::vector<std::vector<u64>> hat_mod;                    // [dst prime index][source]
    };
    BConv make_bconv(const std::vector<int> &src) const {
        BConv bc; bc.src = src; size_t n = src.size();
        bc.hat_inv.resize(n); bc.hat_inv_sh.resize(n);
        for (size_t i = 0; i < n; ++i) {
            const Mod &m = cx.mod[src[i]]; u64 h = 1;
            for (size_t j = 0; j < n; ++j) if (j != i) h = m.mul(h, cx.mod[src[j]].q % m.q);
            bc.hat_inv[i] = m.inv(h); bc.hat_inv_sh[i] = m.shoup(bc.hat_inv[i]);
        }
        bc.hat_mod.assign(cx.nprimes, std::vector<u64>(n, 0));
        for (int t = 0; t < cx.nprimes; ++t) {
            const Mod &m = cx.mod[t];
            for (size_t i = 0; i < n; ++i) {
                u64 h = 1;
                for (size_t j = 0; j < n; ++j) if (j != i) h = m.mul(h, cx.mod[src[j]].q % m.q);
                bc.hat_mod[t][i] = h;
            }
        }
        return bc;
    }

    // Hybrid key switching of one NTT-form polynomial `a` (level+1 limbs).
    //   1. a_c = iNTT(a)
    //   2. per digit b (limbs digit_lo(b) .. digit_hi(b)-1): lift a_c|digit to all of
    //      Q_level u P by fast base conversion (limbs of the digit itself are copied), NTT
    //   3. if g != 0: apply the NTT-domain automorphism to every lifted digit
    //      (decompose-then-permute: the digits of a, not of the permuted a, are lifted,
    //       so several rotations of one ciphertext may share steps 1-2 bit for bit)
    //   4. (c0, c1) = sum_b digit_b (.) key_b   over Q_level u P
    //   5. ModDown: c' = (c - lift_{P->Q}(iNTT(c|P))) * P^-1  on the Q limbs
    void keyswitch(const u64 *a, int level, const Evk &key, u64 g, u64 *out0, u64 *out1) {
        const int N = cx.N, n = level + 1, K = cx.K, ne = n + K, nd = cx.num_digits(level);
        std::vector<u64> ac((size_t)n * N);
#pragma omp parallel for
        for (int l = 0; l < n; ++l) { std::memcpy(&ac[(size_t)l * N], a + (size_t)l * N, N * 8); cx.intt(&ac[(size_t)l * N], l); }
        std::vector<u64> acc0((size_t)ne * N, 0), acc1((size_t)ne * N, 0);
        const std::vector<u32> *perm = g ? &cx.ntt_perm(g) : nullptr;
        for (int dg = 0; dg < nd; ++dg) {
            int lo = cx.digit_lo(dg), hi = cx.digit_hi(dg, n);
            std::vector<int> src; for (int l = lo; l < hi; ++l) src.push_back(l);
            BConv bc = make_bconv(src);
            size_t ns = src.size();
            std::vector<u64> y(ns * N);
            for (size_t i = 0; i < ns; ++i) {
                const Mod &m = cx.mod[src[i]];
                for (int c = 0; c < N; ++c) y[i * N + c] = Mod::mul_shoup(ac[(size_t)src[i] * N + c], bc.hat_inv[i], bc.hat_inv_sh[i], m.q);
            }
#pragma omp parallel for
            for (int j = 0; j < ne; ++j) {
                int pi = cx.prime_index_ext(level, j);
                const Mod &m = cx.mod[pi];
                std::vector<u64> dgt(N);
                if (pi >= lo && pi < hi) {
                    std::memcpy(dgt.data(), a + (size_t)pi * N, N * 8); // already in NTT form
                } else {
                    for (int c = 0; c < N; ++c) {
                        u128 s = 0;
                        for (size_t i = 0; i < ns; ++i) s += (u128)y[i * N + c] * bc.hat_mod[pi][i];
                        dgt[c] = m.red128(s);
                    }
                    cx.ntt(dgt.data(), pi);
                }
                const u64 *k0 = key.limb(dg, 0, pi), *k1 = key.limb(dg, 1, pi);
                u64 *o0 = &acc0[(size_t)j * N], *o1 = &acc1[(size_t)j * N];
                for (int c = 0; c < N; ++c) {
                    u64 v = perm ? dgt[(*perm)[c]] : dgt[c];
                    o0[c] = m.add(o0[c], m.mul(v, k0[c]));
                    o1[c] = m.add(o1[c], m.mul(v, k1[c]));
                }
            }
        }
        // ModDown
        std::vector<int> psrc; for (int j = 0; j < K; ++j) psrc.push_back(cx.L + 1 + j);
        BConv pb = make_bconv(psrc);
        for (int p = 0; p < 2; ++p) {
            std::vector<u64> &acc = p ? acc1 : acc0; u64 *out = p ? out1 : out0;
            std::vector<u64> y((size_t)K * N);
#pragma omp parallel for
            for (int j = 0; j < K; ++j) {
                u64 *pl = &acc[(size_t)(n + j) * N];
                cx.intt(pl, cx.L + 1 + j);
                const Mod &m = cx.mod[cx.L + 1 + j];
                for (int c = 0; c < N; ++c) y[(size_t)j * N + c] = Mod::mul_shoup(pl[c], pb.hat_inv[j], pb.hat_inv_sh[j], m.q);
            }
#pragma omp parallel for
            for (int l = 0; l < n; ++l) {
                const Mod &m = cx.mod[l];
                u64 pinv = 1;
                for (int j = 0; j < K; ++j) pinv = m.mul(pinv, cx.mod[cx.L + 1 + j].q % m.q);
                pinv = m.inv(pinv);
                std::vector<u64> t(N);
                for (int c = 0; c < N; ++c) {
                    u128 s = 0;
                    for (int j = 0; j < K; ++j) s += (u128)y[(size_t)j * N + c] * pb.hat_mod[l][j];
                    t[c] = m.red128(s);
                }
                cx.ntt(t.data(), l);
                const u64 *al = &acc[(size_t)l * N]; u64 *o = out + (size_t)l * N;
                for (int c = 0; c < N; ++c) o[c] = m.mul(m.sub(al[c], t[c]), pinv);
            }
        }
    }

    // Steps 1-2 of keyswitch on their own: the digits of `a` lifted to Q_level u P, NTT form, [digit][ext limb][N].
    std::vector<u64> lifted_digits(const u64 *a, int level) {
        const int N = cx.N, n = level + 1, ne = n + cx.K, nd = cx.num_digits(level);
        std::vector<u64> ac((size_t)n * N), out((size_t)nd * ne * N);
#pragma omp parallel for
        for (int l = 0; l < n; ++l) { std::memcpy(&ac[(size_t)l * N], a + (size_t)l * N, N * 8); cx.intt(&ac[(size_t)l * N], l); }
        for (int dg = 0; dg < nd; ++dg) {
            const int lo = cx.digit_lo(dg), hi = cx.digit_hi(dg, n);
            std::vector<int> src; for (int l = lo; l < hi; ++l) src.push_back(l);
            BConv bc = make_bconv(src);
            const size_t ns = src.size();
            std::vector<u64> y(ns * N);
            for (size_t i = 0; i < ns; ++i)
                for (int c = 0; c < N; ++c) y[i * N + c] = Mod::mul_shoup(ac[(size_t)src[i] * N + c], bc.hat_inv[i], bc.hat_inv_sh[i], cx.mod[src[i]].q);
#pragma omp parallel for
            for (int j = 0; j < ne; ++j) {
                const int pi = cx.prime_index_ext(level, j);
                const Mod &m = cx.mod[pi];
                u64 *d = &out[((size_t)dg * ne + j) * N];
                if (pi >= lo && pi < hi) { std::memcpy(d, a + (size_t)pi * N, N * 8); continue; }
                for (int c = 0; c < N; ++c) {
                    u128 s = 0;
                    for (size_t i = 0; i < ns; ++i) s += (u128)y[i * N + c] * bc.hat_mod[pi][i];
                    d[c] = m.red128(s);
                }
                cx.ntt(d, pi);
            }
        }
        return out;
    }

    // ----- homomorphic primitives -----
    static void require(bool c, const char *msg) { if (!c) throw std::invalid_argument(msg); }

    // HomEvaluator::add / sub / negate (HomEvaluator.hpp:143-146, 222-225, 66-68).
    // Operands of different level: the higher one is brought down with level_down first.
    Ct add(const Ct &x, const Ct &y, bool subtract = false) {
        if (x.level != y.level) {
            if (x.level > y.level) return add(level_down(x, y.level), y, subtract);
            return add(x, level_down(y, x.level), subtract);
        }
        require(x.np == y.np && x.spow == y.spow && x.batch == y.batch, "add: shape mismatch");
        if (count("add", x.level, x.batch)) return meta(x.level, x.np, x.batch, x.spow);
        Ct r = x;
        const int n = x.level + 1, N = cx.N;
#pragma omp parallel for
        for (int i = 0; i < x.batch * x.np * n; ++i) {
            const Mod &m = cx.mod[i % n];
            u64 *o = r.d.data() + (size_t)i * N; const u64 *b = y.d.data() + (size_t)i * N;
            if (subtract) for (int c = 0; c < N; ++c) o[c] = m.sub(o[c], b[c]);
            else for (int c = 0; c < N; ++c) o[c] = m.add(o[c], b[c]);
        }
        return r;
    }
    Ct negate(const Ct &x) {
        if (count("add", x.level, x.batch)) return meta(x.level, x.np, x.batch, x.spow);
        Ct r = x; const int n = x.level + 1, N = cx.N;
        for (int i = 0; i < x.batch * x.np * n; ++i) {
            const Mod &m = cx.mod[i % n]; u64 *o = r.d.data() + (size_t)i * N;
            for (int c = 0; c < N; ++c) o[c] = m.neg(o[c]);
        }
        return r;
    }
    // HomEvaluator::multImagUnit (HomEvaluator.hpp:329-331): multiply by X^(N/2); in NTT form this is
    // +iota on the first half of the limb and -iota on the second half, iota = psi^(N/2).
    Ct mult_imag(const Ct &x) {
        if (count("mult_imag", x.level, x.batch)) return meta(x.level, x.np, x.batch, x.spow);
        Ct r = x; const int n = x.level + 1, N = cx.N;
#pragma omp parallel for
        for (int i = 0; i < x.batch * x.np * n; ++i) {
            int l = i % n; const Mod &m = cx.mod[l]; u64 *o = r.d.data() + (size_t)i * N;
            u64 iu = cx.imag_unit[l], niu = m.neg(iu);
            for (int c = 0; c < N / 2; ++c) o[c] = m.mul(o[c], iu);
            for (int c = N / 2; c < N; ++c) o[c] = m.mul(o[c], niu);
        }
        return r;
    }
    // HomEvaluator::multInteger (HomEvaluator.hpp:346-348)
    Ct mult_int(const Ct &x, i64 k) {
        if (count("mult_imag", x.level, x.batch)) return meta(x.level, x.np, x.batch, x.spow);
        Ct r = x; const int n = x.level + 1, N = cx.N;
#pragma omp parallel for
        for (int i = 0; i < x.batch * x.np * n; ++i) {
            const Mod &m = cx.mod[i % n]; u64 kk = m.from_i64(k); u64 *o = r.d.data() + (size_t)i * N;
            for (int c = 0; c < N; ++c) o[c] = m.mul(o[c], kk);
        }
        return r;
    }
    // HomEvaluator::multWithoutRescale(ct, ptxt) (HomEvaluator.hpp:490-493)
    Ct mul_pt_norescale(const Ct &x, const Pt &p) {
        require(x.level == p.level, "mul_pt: level mismatch");
        require(x.spow == 1 && p.spow == 1, "mul_pt: operand not rescaled");
        if (count("mul_pt", x.level, x.batch)) return meta(x.level, x.np, x.batch, 2);
        Ct r = x; r.spow = 2; const int n = x.level + 1, N = cx.N;
#pragma omp parallel for
        for (int i = 0; i < x.batch * x.np * n; ++i) {
            int l = i % n; const Mod &m = cx.mod[l]; u64 *o = r.d.data() + (size_t)i * N; const u64 *pp = p.limb(l);
            for (int c = 0; c < N; ++c) o[c] = m.mul(o[c], pp[c]);
        }
        return r;
    }
    // HomEvaluator::mult(ct, ptxt) (HomEvaluator.hpp:299-301)
    Ct mul_pt(const Ct &x, const Pt &p) { return rescale(mul_pt_norescale(x, p)); }

    // HomEvaluator::rescale (HomEvaluator.hpp:539-540): drop q_l with rounding.
    //   r = centred lift of the last limb (coefficient form); c_i <- (c_i - r) * q_l^-1 mod q_i
    Ct rescale(const Ct &x) {
        require(x.level >= 1, "rescale: level 0");
        require(x.spow == 2, "rescale: nothing to rescale");
        if (count(x.np == 3 ? "rescale3" : "rescale", x.level, x.batch)) return meta(x.level - 1, x.np, x.batch, 1);
        const int l = x.level, N = cx.N; const u64 ql = cx.mod[l].q;
        Ct r(N, l - 1, x.np, x.batch, 1);
        const int nbp = x.batch * x.np;
        std::vector<u64> lasts((size_t)nbp * N);
#pragma omp parallel for
        for (int bp = 0; bp < nbp; ++bp) {
            std::memcpy(&lasts[(size_t)bp * N], x.limb(bp / x.np, bp % x.np, l), (size_t)N * 8);
            cx.intt(&lasts[(size_t)bp * N], l);
        }
#pragma omp parallel for
        for (int w = 0; w < nbp * l; ++w) {
            const int bp = w / l, i = w % l, b = bp / x.np, p = bp % x.np;
            const u64 *last = &lasts[(size_t)bp * N];
            const Mod &m = cx.mod[i]; u64 qlinv = m.inv(ql % m.q), qlm = ql % m.q;
            std::vector<u64> t(N);
            for (int c = 0; c < N; ++c) {
                u64 v = last[c] % m.q;
                if (last[c] > ql / 2) v = m.sub(v, qlm);
                t[c] = v;
            }
            cx.ntt(t.data(), i);
            const u64 *src = x.limb(b, p, i); u64 *dst = r.limb(b, p, i);
            for (int c = 0; c < N; ++c) dst[c] = m.mul(m.sub(src[c], t[c]), qlinv);
        }
        return r;
    }
    // HomEvaluator::levelDown (HomEvaluator.hpp:574-576): drop limbs to target+1, multiply by the
    // integer round(Delta_target * q_{target+1} / Delta_level), rescale.  Keeps scale = Delta_target.
    Ct level_down(const Ct &x, int target) {
        require(target <= x.level && target >= 0, "level_down: bad target");
        if (target == x.level) return x;
        require(x.spow == 1, "level_down: operand not rescaled");
        const int N = cx.N;
        if (count("scalar_mul", target + 1, x.batch)) return rescale(meta(target + 1, x.np, x.batch, 2));
        Ct t(N, target + 1, x.np, x.batch, 2);
        double cf = cx.scale[target] * (double)cx.mod[target + 1].q / cx.scale[x.level];
        i64 k = (i64)std::rint(cf);
        for (int b = 0; b < x.batch; ++b)
            for (int p = 0; p < x.np; ++p)
                for (int l = 0; l <= target + 1; ++l) {
                    const Mod &m = cx.mod[l]; u64 kk = m.from_i64(k);
                    const u64 *s = x.limb(b, p, l); u64 *o = t.limb(b, p, l);
                    for (int c = 0; c < N; ++c) o[c] = m.mul(s[c], kk);
                }
        return rescale(t);
    }
    // HomEvaluator::tensor (HomEvaluator.hpp:518): (d0,d1,d2) = (b1 b2, a1 b2 + a2 b1, a1 a2)
    Ct tensor(const Ct &x, const Ct &y) {
        require(x.level == y.level && x.np == 2 && y.np == 2 && x.spow == 1 && y.spow == 1 && x.batch == y.batch, "tensor: operands");
        const int n = x.level + 1, N = cx.N;
        if (count("tensor", x.level, x.batch)) return meta(x.level, 3, x.batch, 2);
        Ct r(N, x.level, 3, x.batch, 2);
#pragma omp parallel for collapse(2)
        for (int b = 0; b < x.batch; ++b)
            for (int l = 0; l < n; ++l) {
                const Mod &m = cx.mod[l];
                const u64 *b1 = x.limb(b, 0, l), *a1 = x.limb(b, 1, l), *b2 = y.limb(b, 0, l), *a2 = y.limb(b, 1, l);
                u64 *d0 = r.limb(b, 0, l), *d1 = r.limb(b, 1, l), *d2 = r.limb(b, 2, l);
                for (int c = 0; c < N; ++c) {
                    d0[c] = m.mul(b1[c], b2[c]);
                    d1[c] = m.add(m.mul(a1[c], b2[c]), m.mul(a2[c], b1[c]));
                    d2[c] = m.mul(a1[c], a2[c]);
                }
            }
        return r;
    }
    // HomEvaluator::relinearize (HomEvaluator.hpp:524)
    Ct relin(const Ct &x) {
        require(x.np == 3, "relin: needs 3 polys");
        if (count("relin", x.level, x.batch)) return meta(x.level, 2, x.batch, x.spow);
        const int n = x.level + 1, N = cx.N;
        Ct r(N, x.level, 2, x.batch, x.spow);
        for (int b = 0; b < x.batch; ++b) {
            std::vector<u64> k0((size_t)n * N), k1((size_t)n * N);
            keyswitch(x.limb(b, 2, 0), x.level, mult_key, 0, k0.data(), k1.data());
            for (int l = 0; l < n; ++l) {
                const Mod &m = cx.mod[l];
                for (int c = 0; c < N; ++c) {
                    r.limb(b, 0, l)[c] = m.add(x.limb(b, 0, l)[c], k0[(size_t)l * N + c]);
                    r.limb(b, 1, l)[c] = m.add(x.limb(b, 1, l)[c], k1[(size_t)l * N + c]);
                }
            }
        }
        return r;
    }
    // HomEvaluator::mult(ct, ct) (HomEvaluator.hpp:311-312); operands of different level are aligned
    // by bringing the higher one down first (used by multPackedMatMat, MatrixUtils.cpp:1155)
    Ct mul(const Ct &x, const Ct &y) {
        if (x.level > y.level) return mul(level_down(x, y.level), y);
        if (y.level > x.level) return mul(x, level_down(y, x.level));
        return rescale(relin(tensor(x, y)));
    }

    // automorphism + key switch; g = galois element
    Ct apply_galois(const Ct &x, u64 g) {
        require(x.np == 2, "rotate: needs 2 polys");
        if (g == 1) return x;
        if (count("rotate", x.level, x.batch)) return meta(x.level, 2, x.batch, x.spow);
        auto it = gal_keys.find(g);
        if (it == gal_keys.end()) throw std::runtime_error("missing galois key");
        const int n = x.level + 1, N = cx.N;
        const auto &perm = cx.ntt_perm(g);
        Ct r(N, x.level, 2, x.batch, x.spow);
        for (int b = 0; b < x.batch; ++b) {
            std::vector<u64> k0((size_t)n * N), k1((size_t)n * N);
            keyswitch(x.limb(b, 1, 0), x.level, it->second, g, k0.data(), k1.data());
            for (int l = 0; l < n; ++l) {
                const Mod &m = cx.mod[l]; const u64 *bb = x.limb(b, 0, l);
                for (int c = 0; c < N; ++c) {
                    r.limb(b, 0, l)[c] = m.add(bb[perm[c]], k0[(size_t)l * N + c]);
                    r.limb(b, 1, l)[c] = k1[(size_t)l * N + c];
                }
            }
        }
        return r;
    }
    // The masked sum of two rotations of one ciphertext, rescaled:
    //     p1 (.) rot(x, s1) + p2 (.) rot(x, s2)   ->   level - 1
    // computed with the two key-switch inner products left in the basis Q_level u P, multiplied there by the
    // (extended) plaintexts and summed, and ONE division by D = P * q_level for the sum instead of a ModDown per
    // rotation and a rescale afterwards:
    //   E_p = sum_r p_r (.) (sum_dg perm_r(digit_dg) (.) key_r,dg,p)            over Q_level u P,  p = 0, 1
    //   E_0 += P * sum_r p_r (.) perm_r(c0)                                      on the Q limbs
    //   out_p = (E_p - lift_{D -> Q_{level-1}}(iNTT(E_p | {q_level, P}))) * D^-1  on limbs 0 .. level-1
    // Same slots as rescale(p1 (.) rot + p2 (.) rot); the ciphertext bits differ (one rounding instead of three).
    Ct assemble_rot(const Ct &x, i64 s1, const Pt &p1, i64 s2, const Pt &p2) {
        require(x.np == 2 && x.spow == 1, "assemble_rot: needs a rescaled 2-poly ciphertext");
        require(x.level >= 1, "assemble_rot: level 0");
        require(p1.ext && p2.ext && p1.level == x.level && p2.level == x.level && p1.spow == 1 && p2.spow == 1, "assemble_rot: plaintexts must be extended and at the ciphertext's level");
        const u64 g[2] = {cx.galois_for_rotation(s1), cx.galois_for_rotation(s2)};
        require(g[0] != 1 && g[1] != 1, "assemble_rot: zero rotation");
        if (count("assemble_rot", x.level, x.batch)) return meta(x.level - 1, 2, x.batch, 1);
        const Pt *pp[2] = {&p1, &p2};
        const Evk *key[2]; const std::vector<u32> *perm[2];
        for (int r = 0; r < 2; ++r) {
            auto it = gal_keys.find(g[r]);
            if (it == gal_keys.end()) throw std::runtime_error("missing galois key");
            key[r] = &it->second; perm[r] = &cx.ntt_perm(g[r]);
        }
        const int N = cx.N, level = x.level, n = level + 1, K = cx.K, ne = n + K, nd = cx.num_digits(level);
        std::vector<int> src; src.push_back(level); for (int j = 0; j < K; ++j) src.push_back(cx.L + 1 + j);
        const BConv bc = make_bconv(src);
        const int ns = K + 1;
        Ct out(N, level - 1, 2, x.batch, 1);
        for (int b = 0; b < x.batch; ++b) {
            const std::vector<u64> dg = lifted_digits(x.limb(b, 1, 0), level);
            std::vector<u64> E((size_t)2 * ne * N, 0);
#pragma omp parallel for
            for (int j = 0; j < ne; ++j) {
                const int pi = cx.prime_index_ext(level, j);
                const Mod &m = cx.mod[pi];
                u64 *e0 = &E[(size_t)j * N], *e1 = &E[((size_t)ne + j) * N];
                u64 pmod = 1;
                for (int t = 0; t < K; ++t) pmod = m.mul(pmod, cx.mod[cx.L + 1 + t].q % m.q);
                for (int c = 0; c < N; ++c) {
                    u64 f = 0;
                    for (int r = 0; r < 2; ++r) {
                        const u32 sc = (*perm[r])[c];
                        u64 i0 = 0, i1 = 0;
                        for (int d = 0; d < nd; ++d) {
                            const u64 v = dg[((size_t)d * ne + j) * N + sc];
                            i0 = m.add(i0, m.mul(v, key[r]->limb(d, 0, pi)[c]));
                            i1 = m.add(i1, m.mul(v, key[r]->limb(d, 1, pi)[c]));
                        }
                        const u64 mk = pp[r]->limb(j)[c];
                        e0[c] = m.add(e0[c], m.mul(mk, i0));
                        e1[c] = m.add(e1[c], m.mul(mk, i1));
                        if (j < n) f = m.add(f, m.mul(mk, x.limb(b, 0, j)[sc]));
                    }
                    if (j < n) e0[c] = m.add(e0[c], m.mul(pmod, f));
                }
            }
            for (int p = 0; p < 2; ++p) {
                std::vector<u64> y((size_t)ns * N);
#pragma omp parallel for
                for (int s = 0; s < ns; ++s) {
                    u64 *pl = &E[((size_t)p * ne + (n - 1 + s)) * N];
                    cx.intt(pl, src[s]);
                    for (int c = 0; c < N; ++c) y[(size_t)s * N + c] = Mod::mul_shoup(pl[c], bc.hat_inv[s], bc.hat_inv_sh[s], cx.mod[src[s]].q);
                }
#pragma omp parallel for
                for (int i = 0; i < level; ++i) {
                    const Mod &m = cx.mod[i];
                    u64 dinv = 1;
                    for (int s = 0; s < ns; ++s) dinv = m.mul(dinv, cx.mod[src[s]].q % m.q);
                    dinv = m.inv(dinv);
                    std::vector<u64> t(N);
                    for (int c = 0; c < N; ++c) {
                        u128 acc = 0;
                        for (int s = 0; s < ns; ++s) acc += (u128)y[(size_t)s * N + c] * bc.hat_mod[i][s];
                        t[c] = m.red128(acc);
                    }
                    cx.ntt(t.data(), i);
                    const u64 *e = &E[((size_t)p * ne + i) * N]; u64 *o = out.limb(b, p, i);
                    for (int c = 0; c < N; ++c) o[c] = m.mul(m.sub(e[c], t[c]), dinv);
                }
            }
        }
        return out;
    }
    // Steps 3-4 of keyswitch accumulated into (acc0, acc1) over Q_level u P: acc_p += sum_dg perm_g(digit_dg) (.) key_dg,p
    void ks_inner_acc(const u64 *a, int level, const Evk &key, u64 g, std::vector<u64> &acc0, std::vector<u64> &acc1) {
        const int N = cx.N, n = level + 1, ne = n + cx.K, nd = cx.num_digits(level);
        const std::vector<u64> dg = lifted_digits(a, level);
        const std::vector<u32> *perm = g ? &cx.ntt_perm(g) : nullptr;
#pragma omp parallel for
        for (int j = 0; j < ne; ++j) {
            const int pi = cx.prime_index_ext(level, j);
            const Mod &m = cx.mod[pi];
            u64 *o0 = &acc0[(size_t)j * N], *o1 = &acc1[(size_t)j * N];
            for (int d = 0; d < nd; ++d) {
                const u64 *dv = &dg[((size_t)d * ne + j) * N];
                const u64 *k0 = key.limb(d, 0, pi), *k1 = key.limb(d, 1, pi);
                for (int c = 0; c < N; ++c) {
                    const u64 v = perm ? dv[(*perm)[c]] : dv[c];
                    o0[c] = m.add(o0[c], m.mul(v, k0[c]));
                    o1[c] = m.add(o1[c], m.mul(v, k1[c]));
                }
            }
        }
    }
    // Step 5 of keyswitch on its own: out = (acc - lift_{P->Q}(iNTT(acc|P))) * P^-1 on the Q limbs (acc is consumed)
    void mod_down(std::vector<u64> &acc, int level, u64 *out) {
        const int N = cx.N, n = level + 1, K = cx.K;
        std::vector<int> psrc; for (int j = 0; j < K; ++j) psrc.push_back(cx.L + 1 + j);
        const BConv pb = make_bconv(psrc);
        std::vector<u64> y((size_t)K * N);
#pragma omp parallel for
        for (int j = 0; j < K; ++j) {
            u64 *pl = &acc[(size_t)(n + j) * N];
            cx.intt(pl, cx.L + 1 + j);
            for (int c = 0; c < N; ++c) y[(size_t)j * N + c] = Mod::mul_shoup(pl[c], pb.hat_inv[j], pb.hat_inv_sh[j], cx.mod[cx.L + 1 + j].q);
        }
#pragma omp parallel for
        for (int l = 0; l < n; ++l) {
            const Mod &m = cx.mod[l];
            u64 pinv = 1;
            for (int j = 0; j < K; ++j) pinv = m.mul(pinv, cx.mod[cx.L + 1 + j].q % m.q);
            pinv = m.inv(pinv);
            std::vector<u64> t(N);
            for (int c = 0; c < N; ++c) {
                u128 s = 0;
                for (int j = 0; j < K; ++j) s += (u128)y[(size_t)j * N + c] * pb.hat_mod[l][j];
                t[c] = m.red128(s);
            }
            cx.ntt(t.data(), l);
            const u64 *al = &acc[(size_t)l * N]; u64 *o = out + (size_t)l * N;
            for (int c = 0; c < N; ++c) o[c] = m.mul(m.sub(al[c], t[c]), pinv);
        }
    }
    // sum_i rot(x_i, s_i) with the key-switch inner products of all terms added up in Q_level u P and ONE ModDown
    // for the sum (a rotation by zero adds its operand as it is).  Same slots as the sum of the rotations; the
    // ciphertext bits differ (one rounding instead of one per term).
    Ct rotate_sum(const std::vector<const Ct *> &xs, const std::vector<i64> &steps) {
        require(!xs.empty() && xs.size() == steps.size(), "rotate_sum: nothing to add");
        const Ct &x0 = *xs[0];
        for (const Ct *x : xs) require(x->np == 2 && x->level == x0.level && x->batch == x0.batch && x->spow == x0.spow, "rotate_sum: operands differ in shape");
        if (count("rotate_sum", x0.level, x0.batch * (int)xs.size())) return meta(x0.level, 2, x0.batch, x0.spow);
        const int N = cx.N, level = x0.level, n = level + 1, ne = n + cx.K;
        Ct r(N, level, 2, x0.batch, x0.spow);
        for (int b = 0; b < x0.batch; ++b) {
            std::vector<u64> acc0((size_t)ne * N, 0), acc1((size_t)ne * N, 0), add0((size_t)n * N, 0), add1((size_t)n * N, 0);
            bool switched = false;
            for (size_t i = 0; i < xs.size(); ++i) {
                const u64 g = cx.galois_for_rotation(steps[i]);
                const Ct &x = *xs[i];
                if (g == 1) {
                    for (int l = 0; l < n; ++l) {
                        const Mod &m = cx.mod[l];
                        for (int c = 0; c < N; ++c) {
                            add0[(size_t)l * N + c] = m.add(add0[(size_t)l * N + c], x.limb(b, 0, l)[c]);
                            add1[(size_t)l * N + c] = m.add(add1[(size_t)l * N + c], x.limb(b, 1, l)[c]);
                        }
                    }
                    continue;
                }
                auto it = gal_keys.find(g);
                if (it == gal_keys.end()) throw std::runtime_error("missing galois key");
                ks_inner_acc(x.limb(b, 1, 0), level, it->second, g, acc0, acc1);
                const auto &perm = cx.ntt_perm(g);
                for (int l = 0; l < n; ++l) {
                    const Mod &m = cx.mod[l];
                    for (int c = 0; c < N; ++c) add0[(size_t)l * N + c] = m.add(add0[(size_t)l * N + c], x.limb(b, 0, l)[perm[c]]);
                }
                switched = true;
            }
            std::vector<u64> k0((size_t)n * N, 0), k1((size_t)n * N, 0);
            if (switched) { mod_down(acc0, level, k0.data()); mod_down(acc1, level, k1.data()); }
            for (int l = 0; l < n; ++l) {
                const Mod &m = cx.mod[l];
                for (int c = 0; c < N; ++c) {
                    r.limb(b, 0, l)[c] = m.add(k0[(size_t)l * N + c], add0[(size_t)l * N + c]);
                    r.limb(b, 1, l)[c] = m.add(k1[(size_t)l * N + c], add1[(size_t)l * N + c]);
                }
            }
        }
        return r;
    }
    // HomEvaluator::leftRotate / rightRotate (HomEvaluator.hpp:383, 403): slot p+t moves to slot p
    Ct rotate(const Ct &x, i64 left_steps) { return apply_galois(x, cx.galois_for_rotation(left_steps)); }
    // HomEvaluator::conjugate (HomEvaluator.hpp:465)
    Ct conjugate(const Ct &x) { return apply_galois(x, cx.galois_conj()); }

    // plain NTT over a raw batch of limbs (primitive sweep)
    void ntt_raw(Ct &x, bool inverse) {
        const int n = x.level + 1;
#pragma omp parallel for
        for (int i = 0; i < x.batch * x.np * n; ++i) {
            u64 *p = x.d.data() + (size_t)i * cx.N;
            if (inverse) cx.intt(p, i % n); else cx.ntt(p, i % n);
        }
    }
};

} // namespace orc
