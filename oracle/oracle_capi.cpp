// CPU ORACLE -- TEST INFRASTRUCTURE ONLY (see ckks_oracle.hpp for scope and "parity unpinned").
// C entry points over the oracle, shaped like include/hemmer_b200.h with the prefix orc_,
// so that one test harness can drive the oracle and the CUDA library with the same calls.
#include "ckks_oracle.hpp"
#include "hemmer_oracle.hpp"

using namespace orc;

struct orc_ctx {
    Context cx; Evaluator ev; std::string err;
    explicit orc_ctx(const Params &p) : cx(p), ev(cx) {}
};
typedef Ct orc_ct;
typedef Pt orc_pt;

struct orc_params {
    int32_t log_n, max_level, dnum, num_special, q0_bits, q_bits, p_bits, hamming_weight;
    double sigma; uint64_t seed[4];
};

#define ORC_TRY(ctx, ...)                                                       \
    try { __VA_ARGS__; return 0; }                                                  \
    catch (const std::invalid_argument &e) { (ctx)->err = e.what(); return -1; } \
    catch (const std::runtime_error &e) { (ctx)->err = e.what(); return -4; }    \
    catch (const std::exception &e) { (ctx)->err = e.what(); return -5; }

extern "C" {

int orc_ctx_create(const orc_params *p, int, orc_ctx **out) {
    try {
        Params q; q.log_n = p->log_n; q.max_level = p->max_level; q.dnum = p->dnum; q.num_special = p->num_special;
        q.q0_bits = p->q0_bits; q.q_bits = p->q_bits; q.p_bits = p->p_bits; q.hamming_weight = p->hamming_weight;
        q.sigma = p->sigma; for (int i = 0; i < 4; ++i) q.seed[i] = p->seed[i];
        *out = new orc_ctx(q); return 0;
    } catch (...) { return -1; }
}
void orc_ctx_destroy(orc_ctx *c) { delete c; }
const char *orc_last_error(const orc_ctx *c) { return c->err.c_str(); }
int orc_ctx_info(const orc_ctx *c, uint64_t *primes, double *scales) {
    for (int i = 0; i < c->cx.nprimes; ++i) primes[i] = c->cx.mod[i].q;
    for (int i = 0; i <= c->cx.L; ++i) scales[i] = c->cx.scale[i];
    return 0;
}
int orc_sync(orc_ctx *) { return 0; }
int orc_keygen(orc_ctx *c) { ORC_TRY(c, c->ev.keygen()) }
int orc_gen_rot_keys(orc_ctx *c, const int64_t *steps, int n) { ORC_TRY(c, for (int i = 0; i < n; ++i) c->ev.gen_rot_key(steps[i])) }
uint64_t orc_galois_for_rotation(const orc_ctx *c, int64_t s) { return c->cx.galois_for_rotation(s); }
int orc_evk_export(orc_ctx *c, uint64_t g, uint64_t *host, int *digits) {
    ORC_TRY(c, {
        const Evk *k = nullptr;
        if (g == 0) k = &c->ev.mult_key; else { auto it = c->ev.gal_keys.find(g); if (it == c->ev.gal_keys.end()) throw std::runtime_error("missing key"); k = &it->second; }
        if (digits) *digits = k->nd;
        if (host) std::memcpy(host, k->d.data(), k->d.size() * 8);
    })
}
int orc_secret_export(orc_ctx *c, int64_t *coeff) { std::memcpy(coeff, c->cx.sk_coeff.data(), (size_t)c->cx.N * 8); return 0; }

int orc_encode(orc_ctx *c, const double *re, const double *im, size_t n, int level, orc_pt **out) {
    ORC_TRY(c, {
        std::vector<cplx> z(n);
        for (size_t i = 0; i < n; ++i) z[i] = cplx(re[i], im ? im[i] : 0.0);
        *out = new Pt(c->ev.encode(z.data(), n, level));
    })
}
int orc_encode_ext(orc_ctx *c, const double *re, const double *im, size_t n, int level, orc_pt **out) {
    ORC_TRY(c, {
        std::vector<cplx> z(n);
        for (size_t i = 0; i < n; ++i) z[i] = cplx(re[i], im ? im[i] : 0.0);
        *out = new Pt(c->ev.encode_ext(z.data(), n, level));
    })
}
int orc_decode(orc_ctx *c, const orc_pt *pt, double *re, double *im) {
    ORC_TRY(c, {
        std::vector<cplx> z(c->cx.slots); c->ev.decode(*pt, z.data());
        for (int i = 0; i < c->cx.slots; ++i) { re[i] = z[i].real(); if (im) im[i] = z[i].imag(); }
    })
}
int orc_encrypt(orc_ctx *c, const orc_pt *pt, uint64_t nonce, orc_ct **out) { ORC_TRY(c, *out = new Ct(c->ev.encrypt(*pt, nonce))) }
int orc_decrypt(orc_ctx *c, const orc_ct *ct, int idx, double *re, double *im) {
    ORC_TRY(c, {
        if (ct->d.empty()) throw std::invalid_argument("decrypt: ciphertext produced in dry mode");
        std::vector<cplx> z(c->cx.slots); c->ev.decrypt(*ct, idx, z.data());
        for (int i = 0; i < c->cx.slots; ++i) { re[i] = z[i].real(); if (im) im[i] = z[i].imag(); }
    })
}
int orc_ct_create(orc_ctx *c, int level, int np, int batch, int spow, orc_ct **out) { ORC_TRY(c, *out = new Ct(c->cx.N, level, np, batch, spow, c->ev.dry)) }
int orc_ct_clone(orc_ctx *c, const orc_ct *s, orc_ct **out) { ORC_TRY(c, *out = new Ct(*s)) }
void orc_ct_free(orc_ct *x) { delete x; }
void orc_pt_free(orc_pt *x) { delete x; }
int orc_ct_meta(const orc_ct *x, int *level, int *np, int *batch, int *spow) {
    if (level) *level = x->level; if (np) *np = x->np; if (batch) *batch = x->batch; if (spow) *spow = x->spow; return 0;
}
int orc_pt_meta(const orc_pt *x, int *level, int *spow) { if (level) *level = x->level; if (spow) *spow = x->spow; return 0; }
int orc_ct_import(orc_ctx *, orc_ct *x, const uint64_t *h) { std::memcpy(x->d.data(), h, x->d.size() * 8); return 0; }
int orc_ct_export(orc_ctx *, const orc_ct *x, uint64_t *h) { if (x->d.empty()) return -3; std::memcpy(h, x->d.data(), x->d.size() * 8); return 0; }
int orc_pt_export(orc_ctx *, const orc_pt *x, uint64_t *h) { std::memcpy(h, x->d.data(), x->d.size() * 8); return 0; }
int orc_batch_set(orc_ctx *c, orc_ct *dst, int idx, const orc_ct *src) {
    ORC_TRY(c, {
        Evaluator::require(src->level == dst->level && src->np == dst->np && (idx + 1) * src->batch <= dst->batch, "batch_set");
        if (!src->d.empty() && !dst->d.empty()) std::memcpy(dst->limb(idx * src->batch, 0, 0), src->d.data(), src->d.size() * 8);
    })
}
int orc_batch_get(orc_ctx *c, const orc_ct *src, int idx, orc_ct **out) {
    ORC_TRY(c, {
        Evaluator::require(idx < src->batch, "batch_get");
        Ct *r = new Ct(c->cx.N, src->level, src->np, 1, src->spow, src->d.empty());
        if (!src->d.empty()) std::memcpy(r->d.data(), src->limb(idx, 0, 0), r->d.size() * 8);
        *out = r;
    })
}
int orc_ct_zero(orc_ctx *, orc_ct *x) { std::fill(x->d.begin(), x->d.end(), 0); return 0; }
// single-process stand-ins for the collectives, so that the host-side logic of the multi-rank layer driver can be
// walked through on the CPU (operation bookkeeping in dry mode): nothing is exchanged
int orc_allreduce_sum(orc_ctx *, orc_ct *, void *) { return 0; }
int orc_nccl_group_start() { return 0; }
int orc_nccl_group_end() { return 0; }
int orc_send(orc_ctx *, const orc_ct *, int, void *) { return 0; }
int orc_recv(orc_ctx *, orc_ct *, int, void *) { return 0; }
// exact modular sum of canonical residues (what the owner of a tile computes from the partial products)
int orc_sum_mod_reduce(orc_ctx *c, const orc_ct *const *parts, int count, orc_ct **out) {
    ORC_TRY(c, {
        Evaluator::require(count >= 1 && count <= 16, "sum_mod_reduce");
        Ct *r = new Ct(*parts[0]);
        for (int t = 1; t < count && !r->d.empty(); ++t) {
            Evaluator::require(parts[t]->d.size() == r->d.size(), "sum_mod_reduce: shape");
            const size_t per = (size_t)c->cx.N, limbs = r->d.size() / per, n = (size_t)r->level + 1;
            for (size_t l = 0; l < limbs; ++l) {
                const uint64_t q = c->cx.mod[l % n].q;
                for (size_t i = 0; i < per; ++i) { uint64_t v = r->d[l * per + i] + parts[t]->d[l * per + i]; r->d[l * per + i] = v >= q ? v - q : v; }
            }
        }
        *out = r;
    })
}
int orc_batch_concat(orc_ctx *c, const orc_ct *const *parts, int n, orc_ct **out) {
    ORC_TRY(c, {
        int total = 0;
        for (int k = 0; k < n; ++k) total += parts[k]->batch;
        const bool dry = parts[0]->d.empty();
        Ct *r = new Ct(c->cx.N, parts[0]->level, parts[0]->np, total, parts[0]->spow, dry);
        size_t off = 0;
        if (!dry) for (int k = 0; k < n; ++k) { std::memcpy(r->d.data() + off, parts[k]->d.data(), parts[k]->d.size() * 8); off += parts[k]->d.size(); }
        *out = r;
    })
}
int orc_batch_slice(orc_ctx *c, const orc_ct *src, int start, int count, orc_ct **out) {
    ORC_TRY(c, {
        Evaluator::require(start >= 0 && count >= 1 && start + count <= src->batch, "batch_slice");
        const bool dry = src->d.empty();
        Ct *r = new Ct(c->cx.N, src->level, src->np, count, src->spow, dry);
        if (!dry) std::memcpy(r->d.data(), src->limb(start, 0, 0), r->d.size() * 8);
        *out = r;
    })
}
int orc_add(orc_ctx *c, const orc_ct *a, const orc_ct *b, orc_ct **o) { ORC_TRY(c, *o = new Ct(c->ev.add(*a, *b))) }
int orc_sub(orc_ctx *c, const orc_ct *a, const orc_ct *b, orc_ct **o) { ORC_TRY(c, *o = new Ct(c->ev.add(*a, *b, true))) }
int orc_negate(orc_ctx *c, const orc_ct *a, orc_ct **o) { ORC_TRY(c, *o = new Ct(c->ev.negate(*a))) }
int orc_mult_imag(orc_ctx *c, const orc_ct *a, orc_ct **o) { ORC_TRY(c, *o = new Ct(c->ev.mult_imag(*a))) }
int orc_mult_int(orc_ctx *c, const orc_ct *a, int64_t k, orc_ct **o) { ORC_TRY(c, *o = new Ct(c->ev.mult_int(*a, k))) }
int orc_mul_pt(orc_ctx *c, const orc_ct *a, const orc_pt *p, orc_ct **o) { ORC_TRY(c, *o = new Ct(c->ev.mul_pt(*a, *p))) }
int orc_mul_pt_norescale(orc_ctx *c, const orc_ct *a, const orc_pt *p, orc_ct **o) { ORC_TRY(c, *o = new Ct(c->ev.mul_pt_norescale(*a, *p))) }
int orc_rescale(orc_ctx *c, const orc_ct *a, orc_ct **o) { ORC_TRY(c, *o = new Ct(c->ev.rescale(*a))) }
int orc_level_down(orc_ctx *c, const orc_ct *a, int t, orc_ct **o) { ORC_TRY(c, *o = new Ct(c->ev.level_down(*a, t))) }
int orc_tensor(orc_ctx *c, const orc_ct *a, const orc_ct *b, orc_ct **o) { ORC_TRY(c, *o = new Ct(c->ev.tensor(*a, *b))) }
int orc_relin(orc_ctx *c, const orc_ct *a, orc_ct **o) { ORC_TRY(c, *o = new Ct(c->ev.relin(*a))) }
int orc_mul(orc_ctx *c, const orc_ct *a, const orc_ct *b, orc_ct **o) { ORC_TRY(c, *o = new Ct(c->ev.mul(*a, *b))) }
int orc_rotate(orc_ctx *c, const orc_ct *a, int64_t s, orc_ct **o) { ORC_TRY(c, *o = new Ct(c->ev.rotate(*a, s))) }
int orc_assemble_rot(orc_ctx *c, const orc_ct *a, int64_t s1, const orc_pt *p1, int64_t s2, const orc_pt *p2, orc_ct **o) {
    ORC_TRY(c, *o = new Ct(c->ev.assemble_rot(*a, s1, *p1, s2, *p2)))
}
int orc_rotate_sum(orc_ctx *c, const orc_ct *const *xs, const int64_t *steps, int count, orc_ct **o) {
    ORC_TRY(c, { std::vector<const Ct *> v(xs, xs + count); std::vector<i64> s(steps, steps + count); *o = new Ct(c->ev.rotate_sum(v, s)); })
}
int orc_conjugate(orc_ctx *c, const orc_ct *a, orc_ct **o) { ORC_TRY(c, *o = new Ct(c->ev.conjugate(*a))) }
int orc_ntt(orc_ctx *c, orc_ct *a, int inverse) { ORC_TRY(c, c->ev.ntt_raw(*a, inverse != 0)) }

// plaintext arithmetic (one-polynomial objects)
int orc_pt_mul(orc_ctx *c, const orc_pt *a, const orc_pt *b, orc_pt **o) {
    ORC_TRY(c, { Hemmer h(c->cx, c->ev); *o = new Pt(h.pt_mul(*a, *b)); })
}
int orc_pt_add(orc_ctx *c, const orc_pt *a, const orc_pt *b, orc_pt **o) {
    ORC_TRY(c, { Hemmer h(c->cx, c->ev); *o = new Pt(h.pt_add(*a, *b)); })
}
int orc_pt_rotate(orc_ctx *c, const orc_pt *a, int64_t s, orc_pt **o) {
    ORC_TRY(c, { Hemmer h(c->cx, c->ev); *o = new Pt(h.pt_rotate(*a, s)); })
}

// dry mode and operation counters (see Evaluator::dry)
int orc_set_dry(orc_ctx *c, int on) { c->ev.dry = on != 0; return 0; }
int orc_stats_clear(orc_ctx *c) { c->ev.stats.clear(); return 0; }
// writes "op level count\n" lines; returns the needed buffer size
int orc_stats_dump(orc_ctx *c, char *buf, int cap) {
    std::string s;
    for (auto &kv : c->ev.stats) s += kv.first.first + " " + std::to_string(kv.first.second) + " " + std::to_string(kv.second) + "\n";
    if (buf && cap > 0) { int n = std::min((int)s.size(), cap - 1); std::memcpy(buf, s.data(), n); buf[n] = 0; }
    return (int)s.size() + 1;
}

// --- small self-check helpers used only by the oracle's own unit tests ---
int orc_chacha_block(const uint32_t key[8], uint32_t counter, const uint32_t nonce[3], uint32_t out[16]) {
    uint32_t st[16] = {0x61707865u, 0x3320646eu, 0x79622d32u, 0x6b206574u};
    for (int i = 0; i < 8; ++i) st[4 + i] = key[i];
    st[12] = counter; st[13] = nonce[0]; st[14] = nonce[1]; st[15] = nonce[2];
    ChaCha::core(st, out); return 0;
}
int orc_ntt_limb(orc_ctx *c, uint64_t *a, int prime_index, int inverse) { if (inverse) c->cx.intt(a, prime_index); else c->cx.ntt(a, prime_index); return 0; }
uint64_t orc_psi(const orc_ctx *c, int prime_index) { return c->cx.psi[prime_index][1 << (c->cx.logN - 1)]; } // bitrev(2^(logN-1)) = 1
int orc_ntt_perm(orc_ctx *c, uint64_t g, uint32_t *out) { const auto &p = c->cx.ntt_perm(g); std::memcpy(out, p.data(), p.size() * 4); return 0; }

} // extern "C"

#include "hemmer_capi.inc"
