// Host-side parameter set of the CUDA library: prime chain, NTT twiddles, scale ladder,
// canonical-embedding FFT, key-switch constants and the small host samplers.
// Everything heavy runs on the device; this file only prepares tables and does the
// float64 encode/decode transform (a 2^15-point FFT per plaintext).
//
// Parameter rules (shared with any party that must reproduce the same ciphertext bits):
//   * primes are congruent to 1 modulo 2N.  q_0 is the largest such prime below 2^q0_bits; the K
//     special primes are the next ones below 2^p_bits; the scaling primes q_L..q_1 are picked,
//     top level first, as the unused prime below 2^q_bits closest to Delta_l^2 / 2^q_bits,
//     with Delta_L = 2^q_bits and Delta_{l-1} = Delta_l^2 / q_l evaluated in IEEE double;
//   * psi_q = x^((q-1)/2N) for the least x >= 2 with psi^N = -1;
//   * limb i belongs to key-switch digit (i+1)/alpha, alpha = ceil((L+2)/dnum).
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace hbhost {

typedef unsigned long long u64;
typedef long long i64;
typedef uint32_t u32;
typedef unsigned __int128 u128;

inline u64 mulmod(u64 a, u64 b, u64 q) { return (u64)((u128)a * b % q); }
inline u64 powmod(u64 a, u64 e, u64 q) {
    u64 r = 1; a %= q;
    for (; e; e >>= 1) { if (e & 1) r = mulmod(r, a, q); a = mulmod(a, a, q); }
    return r;
}
inline u64 invmod(u64 a, u64 q) { return powmod(a % q, q - 2, q); }
inline u64 shoup(u64 w, u64 q) { return (u64)(((u128)w << 64) / q); }

// deterministic Miller-Rabin for 64-bit integers
inline bool is_prime(u64 n) {
    static const u64 bases[] = {2, 3, 5, 7, 11, 13, 17, 19, 23, 29, 31, 37};
    if (n < 2) return false;
    for (u64 b : bases) { if (n == b) return true; if (n % b == 0) return false; }
    u64 d = n - 1; int r = 0;
    while (!(d & 1)) { d >>= 1; ++r; }
    for (u64 b : bases) {
        u64 x = powmod(b, d, n);
        if (x == 1 || x == n - 1) continue;
        bool witness = true;
        for (int k = 1; k < r && witness; ++k) { x = mulmod(x, x, n); if (x == n - 1) witness = false; }
        if (witness) return false;
    }
    return true;
}
inline u32 reverse_bits(u32 v, int bits) {
    u32 r = 0;
    for (int k = 0; k < bits; ++k) r |= ((v >> k) & 1u) << (bits - 1 - k);
    return r;
}

struct Cpx { double re, im; };

struct HostParams {
    int log_n, max_level, dnum, num_special, q0_bits, q_bits, p_bits, hamming_weight;
    double sigma;
    u64 seed[4];
};

// ChaCha20 block function (RFC 8439), host copy for the small sequential samplers.
struct HostChaCha {
    u32 key[8];
    static u32 rol(u32 v, int c) { return (v << c) | (v >> (32 - c)); }
    void block(u32 domain, u64 id, u32 counter, u32 out[16]) const {
        u32 s[16] = {0x61707865u, 0x3320646eu, 0x79622d32u, 0x6b206574u, key[0], key[1], key[2], key[3], key[4], key[5], key[6], key[7],
                     counter, domain, (u32)id, (u32)(id >> 32)};
        u32 w[16];
        std::memcpy(w, s, sizeof(w));
#define HBH_Q(a, b, c, d) w[a] += w[b]; w[d] = rol(w[d] ^ w[a], 16); w[c] += w[d]; w[b] = rol(w[b] ^ w[c], 12); \
                          w[a] += w[b]; w[d] = rol(w[d] ^ w[a], 8);  w[c] += w[d]; w[b] = rol(w[b] ^ w[c], 7);
        for (int round = 0; round < 20; round += 2) {
            HBH_Q(0, 4, 8, 12) HBH_Q(1, 5, 9, 13) HBH_Q(2, 6, 10, 14) HBH_Q(3, 7, 11, 15)
            HBH_Q(0, 5, 10, 15) HBH_Q(1, 6, 11, 12) HBH_Q(2, 7, 8, 13) HBH_Q(3, 4, 9, 14)
        }
#undef HBH_Q
        for (int k = 0; k < 16; ++k) out[k] = w[k] + s[k];
    }
    // sequential reader of 64-bit words of one stream
    struct Reader {
        const HostChaCha *c; u32 domain; u64 id; u64 pos; u32 buf[16]; u64 have;
        Reader(const HostChaCha *cc, u32 d, u64 i) : c(cc), domain(d), id(i), pos(0), have(~0ull) {}
        u64 next() {
            u64 blk = pos >> 3;
            if (blk != have) { c->block(domain, id, (u32)blk, buf); have = blk; }
            int k = (int)(pos & 7); ++pos;
            return (u64)buf[2 * k] | ((u64)buf[2 * k + 1] << 32);
        }
    };
};

enum { STREAM_SK = 1, STREAM_ENC_A = 2, STREAM_ENC_E = 3, STREAM_KEY_A = 4, STREAM_KEY_E = 5 };

struct HostCtx {
    HostParams prm;
    int logn, N, slots, L, K, alpha, nprimes;
    std::vector<u64> q;            // [nprimes]
    std::vector<double> scale;     // [L+1]
    std::vector<u64> psi_root;     // [nprimes]
    std::vector<u64> orbit5;       // 5^j mod 2N
    std::vector<Cpx> unit;         // exp(2 pi i k / 2N), k = 0..2N
    std::vector<u64> gauss_cdt;
    HostChaCha cha;

    explicit HostCtx(const HostParams &p) : prm(p) {
        logn = p.log_n; N = 1 << logn; slots = N >> 1; L = p.max_level; K = p.num_special; nprimes = L + 1 + K;
        if (logn < 4 || logn > 16) throw std::invalid_argument("log_n out of range");
        if (L < 1 || K < 1 || K > 8 || nprimes > 32 || p.dnum < 1) throw std::invalid_argument("bad level / special prime count");
        if (p.q0_bits > 60 || p.p_bits > 60 || p.q_bits > 60) throw std::invalid_argument("primes must stay below 2^60");
        if (p.hamming_weight > N || p.hamming_weight < 1) throw std::invalid_argument("bad hamming weight");
        alpha = (L + 2 + p.dnum - 1) / p.dnum;
        if (alpha > 8) throw std::invalid_argument("digit too long");
        const int pbits = K * p.p_bits;
        const int first_digit = p.q0_bits + std::max(0, std::min(alpha - 2, L)) * p.q_bits;
        if (first_digit > pbits || (L + 1 > alpha - 1 && alpha * p.q_bits > pbits))
            throw std::invalid_argument("special modulus narrower than a key-switch digit");
        for (int k = 0; k < 4; ++k) { cha.key[2 * k] = (u32)p.seed[k]; cha.key[2 * k + 1] = (u32)(p.seed[k] >> 32); }
        pick_primes();
        find_roots();
        make_embedding_tables();
        make_gauss_table();
    }

    std::vector<u64> prime_run(int bits, int count) const {
        std::vector<u64> out;
        const u64 step = (u64)2 * N;
        for (u64 c = ((u64)1 << bits) + 1 - step; (int)out.size() < count; c -= step)
            if (is_prime(c)) out.push_back(c);
        return out;
    }
    void pick_primes() {
        q.assign(nprimes, 0);
        q[0] = prime_run(prm.q0_bits, 1)[0];
        std::vector<u64> sp = prime_run(prm.p_bits, K + 1);
        for (int j = 0, t = 0; j < K; ++j) { if (sp[t] == q[0]) ++t; q[L + 1 + j] = sp[t++]; }
        std::vector<u64> pool = prime_run(prm.q_bits, 4 * L + 4);
        std::vector<bool> taken(pool.size(), false);
        scale.assign(L + 1, 0.0);
        const double unit_scale = std::ldexp(1.0, prm.q_bits);
        scale[L] = unit_scale;
        for (int l = L; l > 0; --l) {
            const double want = scale[l] * scale[l] / unit_scale;
            int pick = -1; double gap = 0.0;
            for (size_t c = 0; c < pool.size(); ++c) {
                if (taken[c] || pool[c] == q[0]) continue;
                double g = std::fabs((double)pool[c] - want);
                if (pick < 0 || g < gap) { pick = (int)c; gap = g; }
            }
            taken[pick] = true; q[l] = pool[pick];
            scale[l - 1] = scale[l] * scale[l] / (double)q[l];
        }
    }
    void find_roots() {
        psi_root.assign(nprimes, 0);
        for (int i = 0; i < nprimes; ++i) {
            const u64 e = (q[i] - 1) / ((u64)2 * N);
            for (u64 x = 2; !psi_root[i]; ++x) {
                u64 c = powmod(x, e, q[i]);
                if (powmod(c, (u64)N, q[i]) == q[i] - 1) psi_root[i] = c;
            }
        }
    }
    // twiddle tables of prime i: fwd[k] = psi^bitrev(k), inv[k] = psi^-bitrev(k)
    void twiddles(int i, std::vector<u64> &fwd, std::vector<u64> &fwd_sh, std::vector<u64> &inv, std::vector<u64> &inv_sh) const {
        const u64 m = q[i], r = psi_root[i], ri = invmod(r, m);
        fwd.resize(N); fwd_sh.resize(N); inv.resize(N); inv_sh.resize(N);
        u64 a = 1, b = 1;
        for (int k = 0; k < N; ++k) {
            u32 pos = reverse_bits((u32)k, logn); // power k lands at table slot bitrev(k)
            fwd[pos] = a; fwd_sh[pos] = shoup(a, m);
            inv[pos] = b; inv_sh[pos] = shoup(b, m);
            a = mulmod(a, r, m); b = mulmod(b, ri, m);
        }
    }
    void make_embedding_tables() {
        const u64 M = (u64)2 * N;
        orbit5.resize(slots);
        u64 g = 1;
        for (int j = 0; j < slots; ++j) { orbit5[j] = g; g = g * 5 % M; }
        unit.resize(M + 1);
        const double pi = 3.14159265358979323846264338327950288;
        for (u64 k = 0; k <= M; ++k) {
            const double ang = 2.0 * pi * (double)k / (double)M;
            unit[k].re = std::cos(ang); unit[k].im = std::sin(ang);
        }
    }
    // discrete Gaussian: cdt[k] = floor(2^63 * P(|x| <= k)), magnitudes up to ceil(13 sigma)
    void make_gauss_table() {
        const int J = (int)std::ceil(13.0 * prm.sigma);
        std::vector<double> rho(J + 1);
        for (int j = 0; j <= J; ++j) rho[j] = std::exp(-(double)j * (double)j / (2.0 * prm.sigma * prm.sigma));
        double S = 1.0;
        for (int j = 1; j <= J; ++j) S += 2.0 * rho[j];
        gauss_cdt.resize(J);
        double cum = 0.0;
        for (int k = 0; k < J; ++k) {
            cum += (k == 0 ? rho[0] : 2.0 * rho[k]) / S;
            double v = std::floor(std::ldexp(cum, 63));
            gauss_cdt[k] = v >= 9223372036854775808.0 ? ((u64)1 << 63) : (u64)v;
        }
    }

    int digit_of(int limb) const { return (limb + 1) / alpha; }
    int digit_lo(int d) const { return std::max(0, d * alpha - 1); }
    int digit_hi(int d, int n) const { return std::min((d + 1) * alpha - 1, n); }
    u64 galois_rot(i64 left) const { i64 r = left % slots; if (r < 0) r += slots; return orbit5[(size_t)r]; }
    u64 galois_conj() const { return (u64)2 * N - 1; }

    // ----- special FFT over the orbit of 5 (in place, size = slots) -----
    static void bit_reverse_permute(std::vector<Cpx> &v) {
        const size_t n = v.size();
        for (size_t i = 1, j = 0; i < n; ++i) {
            size_t bit = n >> 1;
            while (j >= bit) { j -= bit; bit >>= 1; }
            j += bit;
            if (i < j) std::swap(v[i], v[j]);
        }
    }
    void embed_inverse(std::vector<Cpx> &v) const { // slot values -> (re, im) halves of the coefficient vector
        const size_t n = v.size(); const u64 M = (u64)2 * N;
        for (size_t len = n; len >= 2; len >>= 1) {
            const size_t h = len >> 1, quad = len << 2; const u64 stride = M / quad;
            for (size_t base = 0; base < n; base += len)
                for (size_t j = 0; j < h; ++j) {
                    const Cpx w = unit[(quad - orbit5[j] % quad) * stride];
                    Cpx a = v[base + j], b = v[base + j + h];
                    Cpx s = {a.re + b.re, a.im + b.im}, d = {a.re - b.re, a.im - b.im};
                    v[base + j] = s;
                    v[base + j + h] = Cpx{d.re * w.re - d.im * w.im, d.re * w.im + d.im * w.re};
                }
        }
        bit_reverse_permute(v);
        const double inv = 1.0 / (double)n;
        for (Cpx &x : v) { x.re = x.re * inv; x.im = x.im * inv; }
    }
    void embed_forward(std::vector<Cpx> &v) const {
        const size_t n = v.size(); const u64 M = (u64)2 * N;
        bit_reverse_permute(v);
        for (size_t len = 2; len <= n; len <<= 1) {
            const size_t h = len >> 1, quad = len << 2; const u64 stride = M / quad;
            for (size_t base = 0; base < n; base += len)
                for (size_t j = 0; j < h; ++j) {
                    const Cpx w = unit[(orbit5[j] % quad) * stride];
                    Cpx a = v[base + j], b = v[base + j + h];
                    Cpx t = {b.re * w.re - b.im * w.im, b.re * w.im + b.im * w.re};
                    v[base + j] = Cpx{a.re + t.re, a.im + t.im};
                    v[base + j + h] = Cpx{a.re - t.re, a.im - t.im};
                }
        }
    }
    // message -> rounded integer coefficients at scale sc
    void encode_coeffs(const double *re, const double *im, size_t n, double sc, std::vector<i64> &coef) const {
        std::vector<Cpx> v((size_t)slots, Cpx{0.0, 0.0});
        for (size_t i = 0; i < n; ++i) { v[i].re = re[i]; v[i].im = im ? im[i] : 0.0; }
        embed_inverse(v);
        coef.resize(N);
        for (int i = 0; i < slots; ++i) {
            coef[i] = (i64)std::rint(v[i].re * sc);
            coef[i + slots] = (i64)std::rint(v[i].im * sc);
        }
    }
    // centred coefficient values (as doubles) -> message
    void decode_values(const std::vector<double> &val, double sc, double *re, double *im) const {
        std::vector<Cpx> v((size_t)slots);
        for (int i = 0; i < slots; ++i) { v[i].re = val[i] / sc; v[i].im = val[i + slots] / sc; }
        embed_forward(v);
        for (int i = 0; i < slots; ++i) { re[i] = v[i].re; if (im) im[i] = v[i].im; }
    }
    // residues of limb 0 (and 1) in coefficient form -> centred doubles
    void centre(const u64 *c0, const u64 *c1, std::vector<double> &val) const {
        val.resize(N);
        if (!c1) {
            for (int i = 0; i < N; ++i) val[i] = c0[i] > q[0] / 2 ? -(double)(q[0] - c0[i]) : (double)c0[i];
            return;
        }
        const u64 q0 = q[0], q1 = q[1], q0inv = invmod(q0 % q1, q1);
        const u128 Q = (u128)q0 * q1;
        for (int i = 0; i < N; ++i) {
            u64 r0 = c0[i], r1 = c1[i], r0m = r0 % q1;
            u64 diff = r1 >= r0m ? r1 - r0m : r1 + q1 - r0m;
            u128 x = (u128)r0 + (u128)q0 * mulmod(diff, q0inv, q1);
            val[i] = x > Q / 2 ? -(double)(__int128)(Q - x) : (double)(__int128)x;
        }
    }

    // ----- host samplers (sequential, small) -----
    void sample_secret(std::vector<i64> &s) const {
        s.assign(N, 0);
        HostChaCha::Reader rd(&cha, STREAM_SK, 0);
        for (int placed = 0; placed < prm.hamming_weight;) {
            u64 r = rd.next();
            size_t pos = (size_t)(r & (u64)(N - 1));
            if (s[pos]) continue;
            s[pos] = (r >> 63) ? -1 : 1; ++placed;
        }
    }
    void sample_gauss(u32 domain, u64 id, std::vector<i64> &e) const {
        e.resize(N);
        HostChaCha::Reader rd(&cha, domain, id);
        for (int c = 0; c < N; ++c) {
            // magnitude = number of table entries <= u; the table is increasing, so stop at the first larger one
            u64 r = rd.next(), u = r >> 1; i64 mag = 0;
            const size_t J = gauss_cdt.size();
            while ((size_t)mag < J && gauss_cdt[(size_t)mag] <= u) ++mag;
            e[c] = (r & 1) ? -mag : mag;
        }
    }
};

} // namespace hbhost
