// Value types and the evaluator facade of the C++ HEMMer layer.
// They stand where HEaaN::Ciphertext / Plaintext / Message / HomEvaluator stand in the reference
// (ciphertext/external/include/HEaaN/{Ciphertext,Plaintext,Message,HomEvaluator}.hpp); every
// operation is one call into the C ABI of include/hemmer_b200.h, i.e. one or more CUDA launches.
#pragma once
#include "hemmer_b200.h"

#include <complex>
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace HELLM {

using i64 = int64_t;
using u64 = uint64_t;
using Complex = std::complex<double>;

// Status codes of the C ABI become the exception types the reference's callers expect:
// std::invalid_argument for level / shape errors (MatrixUtils.cpp:27,36,680,1322),
// std::runtime_error otherwise (utils/check_macros.hpp:49-56).
inline void check(hb_ctx *c, int rc) {
    if (rc == HB_OK) return;
    std::string m = hb_last_error(c);
    if (rc == HB_E_ARG || rc == HB_E_LEVEL || rc == HB_E_SHAPE) throw std::invalid_argument(m);
    throw std::runtime_error(m);
}

// HEaaN::Message: one complex value per slot, kept as two real arrays (the layout hb_encode takes).
struct Message {
    std::vector<double> re, im;
    Message() {}
    explicit Message(size_t n, double v = 0.0) : re(n, v), im(n, 0.0) {}
    size_t size() const { return re.size(); }
    void set(size_t i, Complex v) { re[i] = v.real(); im[i] = v.imag(); }
    // slot s of the result holds slot s - r of the input (HomEvaluator::rightRotate on a Message)
    Message rotated_right(i64 r) const {
        const i64 n = (i64)size();
        r %= n; if (r < 0) r += n;
        Message o(size());
        for (i64 s = 0; s < n; ++s) { i64 d = s + r; if (d >= n) d -= n; o.re[(size_t)d] = re[(size_t)s]; o.im[(size_t)d] = im[(size_t)s]; }
        return o;
    }
};

// HEaaN::Ciphertext (Ciphertext.hpp:29-145).  Copying clones device memory, moving does not.
class Ciphertext {
  public:
    Ciphertext() = default;
    Ciphertext(hb_ctx *c, hb_ct *p) : c_(c), p_(p) {}
    Ciphertext(const Ciphertext &o) : c_(o.c_) { if (o.p_) check(c_, hb_ct_clone(c_, o.p_, &p_)); }
    Ciphertext(Ciphertext &&o) noexcept : c_(o.c_), p_(o.p_) { o.p_ = nullptr; }
    Ciphertext &operator=(Ciphertext o) noexcept { std::swap(c_, o.c_); std::swap(p_, o.p_); return *this; }
    ~Ciphertext() { if (p_) hb_ct_free(p_); }
    hb_ct *raw() const { return p_; }
    hb_ct *release() { hb_ct *p = p_; p_ = nullptr; return p; }
    bool empty() const { return p_ == nullptr; }
    int getLevel() const { int l = -1; hb_ct_meta(p_, &l, nullptr, nullptr, nullptr); return l; }
    int getBatch() const { int b = 0; hb_ct_meta(p_, nullptr, nullptr, &b, nullptr); return b; }
    int getRescaleCounter() const { int s = 1; hb_ct_meta(p_, nullptr, nullptr, nullptr, &s); return s - 1; }
  private:
    hb_ctx *c_ = nullptr;
    hb_ct *p_ = nullptr;
};

// HEaaN::Plaintext.  Plaintexts are immutable once encoded, so copies share the device buffer.
class Plaintext {
  public:
    Plaintext() = default;
    explicit Plaintext(hb_pt *p) : p_(std::make_shared<Holder>(p, true)) {}
    // a handle owned by someone else (kept alive by the caller for the duration of the call)
    static Plaintext borrowed(const hb_pt *p) { Plaintext r; r.p_ = std::make_shared<Holder>(const_cast<hb_pt *>(p), false); return r; }
    hb_pt *raw() const { return p_ ? p_->p : nullptr; }
    // hands the handle to the caller (C entry points); every copy of this Plaintext stops owning it
    hb_pt *release() { if (!p_) return nullptr; p_->owned = false; return p_->p; }
    bool empty() const { return !p_; }
    int getLevel() const { int l = -1; hb_pt_meta(raw(), &l, nullptr); return l; }
  private:
    struct Holder {
        hb_pt *p; bool owned;
        Holder(hb_pt *pp, bool o) : p(pp), owned(o) {}
        ~Holder() { if (owned && p) hb_pt_free(p); }
    };
    std::shared_ptr<Holder> p_;
};

// The step-independent half of a rotation of one ciphertext (lifted key-switch digits), shared by all its rotations.
class Hoisted {
  public:
    Hoisted() = default;
    explicit Hoisted(hb_digits *d) : d_(d, [](hb_digits *x) { hb_digits_free(x); }) {}
    hb_digits *raw() const { return d_.get(); }
  private:
    std::shared_ptr<hb_digits> d_;
};

// A rotation key multiplied once by a mask (or the sum of two), for one level: see hb_masked_key_create.
class MaskedKey {
  public:
    MaskedKey() = default;
    explicit MaskedKey(hb_mkey *k) : k_(k, [](hb_mkey *x) { hb_masked_key_free(x); }) {}
    hb_mkey *raw() const { return k_.get(); }
    bool empty() const { return !k_; }
  private:
    std::shared_ptr<hb_mkey> k_;
};

// The subset of HEaaN::HomEvaluator / EnDecoder the matmul path uses (HomEvaluator.hpp:30-616).
class Evaluator {
  public:
    explicit Evaluator(hb_ctx *c) : c_(c) {}
    hb_ctx *ctx() const { return c_; }

    Plaintext encode(const Message &m, int level) const {
        hb_pt *p = nullptr; check(c_, hb_encode(c_, m.re.data(), m.im.data(), m.size(), level, &p)); return Plaintext(p);
    }
    Plaintext encodeExtended(const Message &m, int level) const {
        hb_pt *p = nullptr; check(c_, hb_encode_ext(c_, m.re.data(), m.im.data(), m.size(), level, &p)); return Plaintext(p);
    }
    Message decode(const Plaintext &p, size_t slots) const {
        Message m(slots); check(c_, hb_decode(c_, p.raw(), m.re.data(), m.im.data())); return m;
    }
#define HB_UNARY(name, fn) Ciphertext name(const Ciphertext &a) const { hb_ct *o = nullptr; check(c_, fn(c_, a.raw(), &o)); return Ciphertext(c_, o); }
#define HB_BINARY(name, fn) Ciphertext name(const Ciphertext &a, const Ciphertext &b) const { hb_ct *o = nullptr; check(c_, fn(c_, a.raw(), b.raw(), &o)); return Ciphertext(c_, o); }
    HB_BINARY(add, hb_add)
    HB_BINARY(sub, hb_sub)
    HB_BINARY(tensor, hb_tensor)
    HB_BINARY(mult, hb_mul)
    Ciphertext multInteger(const Ciphertext &a, i64 k) const { hb_ct *o = nullptr; check(c_, hb_mult_int(c_, a.raw(), k, &o)); return Ciphertext(c_, o); }
    Ciphertext square(const Ciphertext &a) const { hb_ct *o = nullptr; check(c_, hb_square(c_, a.raw(), &o)); return Ciphertext(c_, o); }
    HB_UNARY(negate, hb_negate)
    HB_UNARY(multImagUnit, hb_mult_imag)
    HB_UNARY(rescale, hb_rescale)
    HB_UNARY(relinearize, hb_relin)
    HB_UNARY(conjugate, hb_conjugate)
#undef HB_UNARY
#undef HB_BINARY
    Ciphertext mult(const Ciphertext &a, const Plaintext &p) const { hb_ct *o = nullptr; check(c_, hb_mul_pt(c_, a.raw(), p.raw(), &o)); return Ciphertext(c_, o); }
    Ciphertext multWithoutRescale(const Ciphertext &a, const Plaintext &p) const {
        hb_ct *o = nullptr; check(c_, hb_mul_pt_norescale(c_, a.raw(), p.raw(), &o)); return Ciphertext(c_, o);
    }
    Ciphertext levelDown(const Ciphertext &a, int target) const { hb_ct *o = nullptr; check(c_, hb_level_down(c_, a.raw(), target, &o)); return Ciphertext(c_, o); }
    Ciphertext levelDownOne(const Ciphertext &a) const { return levelDown(a, a.getLevel() - 1); }
    // one direct switching key per step, generated on first use (the reference composes power-of-two keys)
    Ciphertext leftRotate(const Ciphertext &a, i64 steps) const {
        check(c_, hb_gen_rot_keys(c_, &steps, 1));
        hb_ct *o = nullptr; check(c_, hb_rotate(c_, a.raw(), steps, &o)); return Ciphertext(c_, o);
    }
    Ciphertext rightRotate(const Ciphertext &a, i64 steps) const { return leftRotate(a, -steps); }
    // many rotations of one ciphertext: decompose once, then one cheap call per step (same bits as leftRotate)
    Hoisted decompose(const Ciphertext &a) const { hb_digits *d = nullptr; check(c_, hb_decompose(c_, a.raw(), &d)); return Hoisted(d); }
    Ciphertext leftRotate(const Ciphertext &a, const Hoisted &h, i64 steps) const {
        check(c_, hb_gen_rot_keys(c_, &steps, 1));
        hb_ct *o = nullptr; check(c_, hb_rotate_hoisted(c_, a.raw(), h.raw(), steps, &o)); return Ciphertext(c_, o);
    }
    // sum_t leftRotate(x[t], steps[t]) with one ModDown for the whole sum
    Ciphertext rotateSum(const std::vector<Ciphertext> &x, const std::vector<i64> &steps) const {
        check(c_, hb_gen_rot_keys(c_, steps.data(), (int)steps.size()));
        std::vector<const hb_ct *> raw;
        for (const auto &v : x) raw.push_back(v.raw());
        hb_ct *o = nullptr; check(c_, hb_rotate_sum(c_, raw.data(), steps.data(), (int)raw.size(), &o)); return Ciphertext(c_, o);
    }
    Plaintext mult(const Plaintext &a, const Plaintext &b) const { hb_pt *o = nullptr; check(c_, hb_pt_mul(c_, a.raw(), b.raw(), &o)); return Plaintext(o); }
    Plaintext add(const Plaintext &a, const Plaintext &b) const { hb_pt *o = nullptr; check(c_, hb_pt_add(c_, a.raw(), b.raw(), &o)); return Plaintext(o); }
    Plaintext leftRotate(const Plaintext &p, i64 steps) const { hb_pt *o = nullptr; check(c_, hb_pt_rotate(c_, p.raw(), steps, &o)); return Plaintext(o); }
    // rescale(a (.) pa + b (.) pb): the "assemble" step of the matmul loops in one pass
    Ciphertext assemble(const Ciphertext &a, const Plaintext &pa, const Ciphertext &b, const Plaintext &pb) const {
        hb_ct *o = nullptr; check(c_, hb_mul2_add_rescale(c_, a.raw(), pa.raw(), b.raw(), pb.raw(), &o)); return Ciphertext(c_, o);
    }
    // pa (.) rot(a, sa) + pb (.) rot(a, sb), one level down: both key switches stay in the extended basis and share
    // one division by P * q_level (pa, pb from encodeExtended)
    Ciphertext assembleRotations(const Ciphertext &a, const Hoisted &h, i64 sa, const Plaintext &pa, i64 sb, const Plaintext &pb) const {
        const i64 steps[2] = {sa, sb};
        check(c_, hb_gen_rot_keys(c_, steps, 2));
        hb_ct *o = nullptr; check(c_, hb_assemble_hoisted(c_, a.raw(), h.raw(), sa, pa.raw(), sb, pb.raw(), &o)); return Ciphertext(c_, o);
    }
    // the same from rotation keys that already carry the masks; kb may be empty (one masked rotation)
    MaskedKey maskedKey(i64 steps, const Plaintext &m1, const Plaintext *m2 = nullptr) const {
        check(c_, hb_gen_rot_keys(c_, &steps, 1));
        hb_mkey *k = nullptr; check(c_, hb_masked_key_create(c_, steps, m1.raw(), m2 ? m2->raw() : nullptr, &k)); return MaskedKey(k);
    }
    Ciphertext assembleRotations(const Ciphertext &a, const Hoisted &h, const MaskedKey &ka, const MaskedKey &kb) const {
        hb_ct *o = nullptr; check(c_, hb_assemble_masked(c_, a.raw(), h.raw(), ka.raw(), kb.raw(), &o)); return Ciphertext(c_, o);
    }
    // several wrapped copies of the same input in one launch sequence; member g * batch + b of the result is copy g of input b
    Ciphertext assembleRotationsMulti(const Ciphertext &a, const Hoisted &h, const std::vector<const MaskedKey *> &ka, const std::vector<const MaskedKey *> &kb) const {
        std::vector<const hb_mkey *> k1, k2;
        for (size_t g = 0; g < ka.size(); ++g) { k1.push_back(ka[g]->raw()); k2.push_back(kb[g] ? kb[g]->raw() : nullptr); }
        hb_ct *o = nullptr; check(c_, hb_assemble_masked_multi(c_, a.raw(), h.raw(), k1.data(), k2.data(), (int)k1.size(), &o)); return Ciphertext(c_, o);
    }
    // acc += sum_g tensor(a[g], b[g]) for group-major batches of `groups` groups
    void tensorAccumulateGroups(Ciphertext &acc, const Ciphertext &a, const Ciphertext &b, int groups) const {
        hb_ct *p = acc.release();
        int rc = hb_tensor_acc_groups(c_, a.raw(), b.raw(), groups, &p);
        acc = Ciphertext(c_, p);
        check(c_, rc);
    }
    Ciphertext concat(const std::vector<Ciphertext> &parts) const {
        std::vector<const hb_ct *> raw;
        for (const auto &x : parts) raw.push_back(x.raw());
        hb_ct *o = nullptr; check(c_, hb_batch_concat(c_, raw.data(), (int)raw.size(), &o)); return Ciphertext(c_, o);
    }
    // sum_j mult(a[j], p[j]): every product is rescaled as eval.mult(ct, mask) does, the results are added
    Ciphertext multSum(const std::vector<const Ciphertext *> &a, const std::vector<const Plaintext *> &p) const {
        std::vector<const hb_ct *> ra; std::vector<const hb_pt *> rp;
        for (auto *x : a) ra.push_back(x->raw());
        for (auto *x : p) rp.push_back(x->raw());
        hb_ct *o = nullptr; check(c_, hb_mul_pt_sum(c_, ra.data(), rp.data(), (int)ra.size(), &o)); return Ciphertext(c_, o);
    }
    // rescale(sum_j multWithoutRescale(a[j], p[j])): one rescale for the whole sum
    Ciphertext multSumRescaledOnce(const std::vector<const Ciphertext *> &a, const std::vector<const Plaintext *> &p) const {
        std::vector<const hb_ct *> ra; std::vector<const hb_pt *> rp;
        for (auto *x : a) ra.push_back(x->raw());
        for (auto *x : p) rp.push_back(x->raw());
        hb_ct *o = nullptr; check(c_, hb_sum_mul_pt_rescale(c_, ra.data(), rp.data(), (int)ra.size(), &o)); return Ciphertext(c_, o);
    }
    // all giant-step parts of a baby-step / giant-step transform in one pass over the shared terms:
    // part g = rescale(sum_j multWithoutRescale(a[j], p[g][j])), null entries skipped; members part-major in the result
    static constexpr size_t kMaxPartTerms = 17, kMaxParts = 17;
    Ciphertext multSumRescaledOnceParts(const std::vector<const Ciphertext *> &a, const std::vector<std::vector<const Plaintext *>> &p) const {
        std::vector<const hb_ct *> ra; std::vector<const hb_pt *> rp;
        for (auto *x : a) ra.push_back(x->raw());
        for (const auto &row : p)
            for (size_t j = 0; j < a.size(); ++j) rp.push_back(j < row.size() && row[j] ? row[j]->raw() : nullptr);
        hb_ct *o = nullptr; check(c_, hb_mul_pt_sum_parts(c_, ra.data(), rp.data(), (int)ra.size(), (int)p.size(), &o)); return Ciphertext(c_, o);
    }
    // sum_t leftRotate(member group t of x, steps[t]) with one lift of the digits and one ModDown
    Ciphertext rotateSumGrouped(const Ciphertext &x, const std::vector<i64> &steps) const {
        check(c_, hb_gen_rot_keys(c_, steps.data(), (int)steps.size()));
        hb_ct *o = nullptr; check(c_, hb_rotate_sum_grouped(c_, x.raw(), steps.data(), (int)steps.size(), &o)); return Ciphertext(c_, o);
    }
    // acc += tensor(a, b)
    void tensorAccumulate(Ciphertext &acc, const Ciphertext &a, const Ciphertext &b) const {
        hb_ct *p = acc.release();
        int rc = hb_tensor_acc(c_, a.raw(), b.raw(), &p);
        acc = Ciphertext(c_, p);
        check(c_, rc);
    }
    // HomEvaluator::matmul (HomEvaluator.hpp:595-601)
    Ciphertext matmul(const Ciphertext &pre, const Plaintext &pt, i64 row_step) const {
        hb_ct *o = nullptr; check(c_, hb_matmul_acc(c_, pre.raw(), pt.raw(), row_step, &o)); return Ciphertext(c_, o);
    }
    // sum over the K-groups b0 .. b0+pts.size()-1 of a batched set of shifted copies
    Ciphertext matmulGroups(const Ciphertext &pre, int btotal, int b0, const std::vector<const hb_pt *> &pts, i64 row_step) const {
        hb_ct *o = nullptr; check(c_, hb_matmul_acc_multi(c_, pre.raw(), btotal, b0, pts.data(), (int)pts.size(), row_step, &o)); return Ciphertext(c_, o);
    }
    Ciphertext stack(const std::vector<Ciphertext> &v) const {
        int level = 0, np = 0, sp = 0, b = 1; hb_ct_meta(v[0].raw(), &level, &np, &b, &sp);
        hb_ct *o = nullptr; check(c_, hb_ct_create(c_, level, np, (int)v.size() * b, sp, &o)); // copy k of input j at k*b + j
        Ciphertext out(c_, o);
        for (size_t k = 0; k < v.size(); ++k) check(c_, hb_batch_set(c_, o, (int)k, v[k].raw()));
        return out;
    }
    Ciphertext slice(const Ciphertext &b, int k) const { hb_ct *o = nullptr; check(c_, hb_batch_get(c_, b.raw(), k, &o)); return Ciphertext(c_, o); }
  private:
    hb_ctx *c_;
};

} // namespace HELLM
