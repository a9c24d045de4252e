// HELLM::HEMMer methods: slot layouts, encrypt / decrypt, packing helpers, and the entry points
// that forward to the schedules (the role of ciphertext/src/HEMMer.cpp on the matmul path).
#include "HEMMer.hpp"
#include "schedules.hpp"

namespace HELLM {

namespace {
enum HemmerMask { kColEven = 1, kRowEven = 2, kLeftHalf = 3, kLeftHalfScaled = 4, kFirstCol = 5, kLastCol = 6, kFirstRow = 7, kFirstColOnly = 8, kHeadLeft = 9, kHeadRight = 10, kRightHalf = 11 };
}

HEMMer::HEMMer(hb_ctx *ctx) : ctx_(ctx), eval_(ctx) {
    int log_n = 0, L = 0;
    hb_ctx_dims(ctx, &log_n, &L, nullptr);
    slots_ = (i64)1 << (log_n - 1);
    max_level_ = L;
    tile_ = 1;
    while (2 * tile_ * tile_ < slots_) tile_ <<= 1; // side of the tile two of which fill a ciphertext
}
HEMMer *HEMMer::genHEMMer(int device_id, const hb_params &prm) {
    hb_ctx *c = nullptr;
    if (hb_ctx_create(&prm, device_id, &c) != HB_OK) throw std::runtime_error("[genHEMMer] cannot create a context on this device");
    int rc = hb_keygen(c);
    if (rc != HB_OK) { std::string m = hb_last_error(c); hb_ctx_destroy(c); throw std::runtime_error(m); }
    HEMMer *h = new HEMMer(c);
    h->owns_ctx_ = true;
    return h;
}
HEMMer::~HEMMer() {
    masks_.clear();
    if (owns_ctx_) hb_ctx_destroy(ctx_);
}

// ---- layouts ----
// HEMMer::message2 (HEMMer.cpp:249-261): [A | B], row-major
Message HEMMer::message2(const double *d1, const double *d2, i64 h, i64 w) const {
    if (h * 2 * w > slots_) throw std::invalid_argument("[message2] matrices do not fit the slots");
    Message m((size_t)slots_);
    for (i64 r = 0; r < h; ++r)
        for (i64 c = 0; c < w; ++c) {
            m.re[(size_t)(r * 2 * w + c)] = d1[r * w + c];
            m.re[(size_t)(r * 2 * w + w + c)] = d2[r * w + c];
        }
    return m;
}
// HEMMer::msgDiagonalToRow4 (HEMMer.cpp:353-398): left half 1/2 (W1 - i W3), right half 1/2 (W2 - i W4),
// every column j rolled up by j rows (the cleartext tau transform)
Message HEMMer::msgDiagonalToRow4(const double *w1, const double *w2, const double *w3, const double *w4, i64 h, i64 w) const {
    if (h * 2 * w > slots_) throw std::invalid_argument("[msgDiagonalToRow4] matrices do not fit the slots");
    Message m((size_t)slots_);
    for (i64 r = 0; r < h; ++r)
        for (i64 c = 0; c < w; ++c) {
            const i64 src = ((r + c) % h) * w + c;
            m.set((size_t)(r * 2 * w + c), Complex(0.5 * w1[src], -0.5 * w3[src]));
            m.set((size_t)(r * 2 * w + w + c), Complex(0.5 * w2[src], -0.5 * w4[src]));
        }
    return m;
}
PtxtTensor HEMMer::encode(const double *data, i64 h, i64 w, int level) const {
    if (h * w > slots_) throw std::invalid_argument("[encode] matrix does not fit the slots");
    Message m((size_t)slots_);
    for (i64 i = 0; i < h * w; ++i) m.re[(size_t)i] = data[i];
    return PtxtTensor(h, w, eval_.encode(m, level ? level : max_level_));
}
PtxtTensor HEMMer::encode2(const double *d1, const double *d2, i64 h, i64 w, int level) const {
    return PtxtTensor(h, w, eval_.encode(message2(d1, d2, h, w), level ? level : max_level_), 2 * w);
}
PtxtTensor HEMMer::encodeDiagonalToRow4(const double *w1, const double *w2, const double *w3, const double *w4, i64 h, i64 w, int level) const {
    return PtxtTensor(h, w, eval_.encode(msgDiagonalToRow4(w1, w2, w3, w4, h, w), level ? level : max_level_), 2 * w);
}
CtxtTensor HEMMer::encrypt(const double *data, i64 h, i64 w, u64 nonce) const {
    PtxtTensor p = encode(data, h, w);
    hb_ct *ct = nullptr;
    check(ctx_, hb_encrypt(ctx_, p.get().raw(), nonce, &ct));
    return CtxtTensor(p.getShape(), Ciphertext(ctx_, ct));
}
CtxtTensor HEMMer::encrypt2(const double *d1, const double *d2, i64 h, i64 w, u64 nonce) const {
    PtxtTensor p = encode2(d1, d2, h, w);
    hb_ct *ct = nullptr;
    check(ctx_, hb_encrypt(ctx_, p.get().raw(), nonce, &ct));
    return CtxtTensor(p.getShape(), Ciphertext(ctx_, ct));
}
void HEMMer::decrypt(const CtxtTensor &t, double *out) const {
    std::vector<double> re((size_t)slots_), im((size_t)slots_);
    check(ctx_, hb_decrypt(ctx_, t.get().raw(), 0, re.data(), im.data()));
    for (i64 i = 0; i < t.getHeight() * t.getWidth(); ++i) out[i] = re[(size_t)i];
}
void HEMMer::decrypt2(const CtxtTensor &t, double *out) const {
    std::vector<double> re((size_t)slots_), im((size_t)slots_);
    check(ctx_, hb_decrypt(ctx_, t.get().raw(), 0, re.data(), im.data()));
    const i64 h = t.getHeight(), w = t.getWidth();
    for (i64 r = 0; r < h; ++r)
        for (i64 c = 0; c < w; ++c) {
            out[r * w + c] = re[(size_t)(r * 2 * w + c)];
            out[h * w + r * w + c] = re[(size_t)(r * 2 * w + w + c)];
        }
}
void HEMMer::addInplace(CtxtTensor &a, const CtxtTensor &b) const { a.get() = eval_.add(a.get(), b.get()); }
void HEMMer::hadamardMultInplace(CtxtTensor &a, const CtxtTensor &b) const { a.get() = eval_.mult(a.get(), b.get()); }
void HEMMer::hadamardMultInplace(CtxtTensor &a, const PtxtTensor &b) const { a.get() = eval_.mult(a.get(), b.get()); }
void HEMMer::save(const std::string &keys_path) const { check(ctx_, hb_keys_save(ctx_, keys_path.c_str())); }

// ---- schedules ----
#define HB_ENV sched::Env env{eval_, slots_, masks_, schedule_}
CtxtTensor HEMMer::singleCCMatMul(const CtxtTensor &a, const CtxtTensor &b, int t) { HB_ENV; return sched::multMatMatCC(env, a, b, t); }
CtxtTensor HEMMer::singleMatMul(const CtxtTensor &a, const PtxtTensor &b, int t) { HB_ENV; return sched::multMatMatCP(env, a, b, t); }
void HEMMer::ccMatMulPrepare(const CtxtTensor &a, const CtxtTensor &b, int t, Ciphertext &sa, Ciphertext &tb) { HB_ENV; sched::ccmmPrepare(env, a, b, t, sa, tb); }
CtxtTensor HEMMer::ccMatMulCore(Ciphertext sa, Ciphertext tb, i64 rows, i64 inner, i64 cols, i64 width, int t) {
    HB_ENV; return sched::ccmmCore(env, std::move(sa), std::move(tb), rows, inner, cols, width, t);
}
CtxtTensor HEMMer::packedMatMul(const CtxtTensor &a, const CtxtTensor &b, int t) { HB_ENV; return sched::multPackedMatMat(env, a, b, t); }
CtxtTensor HEMMer::packedMatMulPre(const CtxtTensor &a, int t) { HB_ENV; return sched::multPackedMatMatPre(env, a, t); }
Ciphertext HEMMer::packedMatMulPreRot(const CtxtTensor &a, int t) { HB_ENV; return sched::multPackedMatMatPreRot(env, a, t); }
CtxtTensor HEMMer::packedMatMulPreRev(const CtxtTensor &b, int t) { HB_ENV; return sched::multPackedMatMatPreRev(env, b, t); }
CtxtTensor HEMMer::packedMatMulCCReuse(const Ciphertext &pre, const CtxtTensor &b, int) { HB_ENV; return sched::multPackedMatMatCCReuse(env, pre, b); }
Ciphertext HEMMer::matMulPre(const CtxtTensor &a, int t) { HB_ENV; return sched::multMatMatPre(env, a, t); }
CtxtTensor HEMMer::matMulReUse(const Ciphertext &pre, const PtxtTensor &w, int) { HB_ENV; return sched::multMatMatReUse(env, pre, w); }
CtxtTensor HEMMer::matMulPreRev(const CtxtTensor &b, int t) { HB_ENV; return sched::multMatMatPreRev(env, b, t); }
CtxtTensor HEMMer::matMulCCReUse(const Ciphertext &pre, const CtxtTensor &b, int) { HB_ENV; return sched::multMatMatCCReUse(env, pre, b); }
CtxtTensor HEMMer::diagonalToColumn(const CtxtTensor &t) { HB_ENV; return sched::diagonalToColumn(env, t); }
CtxtTensor HEMMer::diagonalToRow(const CtxtTensor &t) { HB_ENV; return sched::diagonalToRow(env, t); }

// HEMMer::transposeInplace -- HEMMer.cpp:1166-1172
void HEMMer::transposeInplace(CtxtTensor &t, int target_level) {
    HB_ENV;
    if (target_level > 0) t.get() = eval_.levelDown(t.get(), 1 + target_level);
    t = sched::transpose(env, t);
}

// ---- packing helpers: masks over two side-by-side tiles (generateAxisMasks / generateRightLeftMasks,
// HEMMer.cpp:2345-2393), encoded per level on first use ----
static const Plaintext &hemmer_mask(HEMMer &h, int which, int level) {
    MaskCache::Key k{sched::kHemmer, TileTensorShape(h.tile(), h.tile(), 2 * h.tile()), which, level};
    if (const Plaintext *p = h.masks().find(k)) return *p;
    const i64 d = h.tile();
    if (2 * d * d != h.slots()) throw std::invalid_argument("[HEMMer] slot count is not 2*d^2: tile packing unavailable");
    Message m((size_t)h.slots());
    for (i64 r = 0; r < d; ++r)
        for (i64 c = 0; c < 2 * d; ++c) {
            bool on = which == kColEven ? ((c % d) % 2 == 0) : which == kRowEven ? (r % 2 == 0) : which == kFirstCol ? (c % d == 0) : which == kLastCol ? (c % d == d - 1) :
                      which == kFirstRow ? (r == 0) : which == kFirstColOnly ? (c == 0) :
                      which == kHeadLeft ? (c % d < d / 2) : which == kHeadRight ? (c % d >= d / 2) : which == kRightHalf ? (c >= d) : (c < d);
            if (on) m.re[(size_t)(r * 2 * d + c)] = which == kLeftHalfScaled ? 0.5 : 1.0;
        }
    return h.masks().put(k, h.eval().encode(m, level));
}
// shared body of complexPackingInplace (HEMMer.cpp:764-777), transposeComplexPackingInplace (:779-799, first half)
// and complexPackingRowInplace (:801-817): fold odd columns (rows) into the imaginary part of the even ones
static Ciphertext fold_odd(HEMMer &h, const Ciphertext &x, int mask, i64 step, bool negate, bool even_first) {
    const Evaluator &ev = h.eval();
    Ciphertext even = ev.mult(x, hemmer_mask(h, mask, x.getLevel()));
    Ciphertext odd = ev.multImagUnit(ev.leftRotate(x, step));
    if (negate) odd = ev.negate(odd);
    odd = ev.mult(odd, hemmer_mask(h, mask, odd.getLevel()));
    Ciphertext fus = even_first ? ev.add(even, odd) : ev.add(odd, even);
    return ev.add(ev.rightRotate(fus, step), fus);
}
void HEMMer::complexPackingInplace(CtxtTensor &t) { t.get() = fold_odd(*this, t.get(), kColEven, 1, false, false); }
void HEMMer::transposeComplexPackingInplace(CtxtTensor &t, int target_level) {
    t.get() = fold_odd(*this, t.get(), kColEven, 1, true, false);
    if (target_level > 0) t.get() = eval_.levelDown(t.get(), 1 + target_level);
    transposeInplace(t, 0);
}
void HEMMer::complexPackingRowInplace(CtxtTensor &t) { t.get() = fold_odd(*this, t.get(), kRowEven, t.getBlockWidth(), true, true); }
// HEMMer::oneMatRotSumInplace -- HEMMer.cpp:882-919 with ModelArgs::HEAD_DIM equal to the tile side
void HEMMer::oneMatRotSumInplace(CtxtTensor &a, CtxtTensor &b) {
    const i64 d = tile_;
    for (i64 rot = 1; rot < d / 2; rot <<= 1) {
        a.get() = eval_.add(a.get(), eval_.leftRotate(a.get(), rot));
        b.get() = eval_.add(b.get(), eval_.rightRotate(b.get(), rot));
    }
    a.get() = eval_.mult(a.get(), hemmer_mask(*this, kFirstCol, a.getLevel()));
    b.get() = eval_.mult(b.get(), hemmer_mask(*this, kLastCol, b.getLevel()));
    for (i64 rot = 1; rot < d; rot <<= 1) {
        a.get() = eval_.add(a.get(), eval_.rightRotate(a.get(), rot));
        b.get() = eval_.add(b.get(), eval_.leftRotate(b.get(), rot));
    }
}
// HEMMer::tr_oneMatRotSumInplace -- HEMMer.cpp:921-962 with ModelArgs::HEAD_DIM equal to the tile side: the sums run over a
// whole row of a tile and come back on half of it (a: left half, b: right half), after an optional level-down
void HEMMer::trOneMatRotSumInplace(CtxtTensor &a, CtxtTensor &b, int target_level) {
    const i64 d = tile_;
    if (target_level > 0) {
        a.get() = eval_.levelDown(a.get(), target_level + 1);
        b.get() = eval_.levelDown(b.get(), target_level + 1);
    }
    for (i64 rot = 1; rot < d; rot <<= 1) {
        a.get() = eval_.add(a.get(), eval_.leftRotate(a.get(), rot));
        b.get() = eval_.add(b.get(), eval_.rightRotate(b.get(), rot));
    }
    a.get() = eval_.mult(a.get(), hemmer_mask(*this, kFirstCol, a.getLevel()));
    b.get() = eval_.mult(b.get(), hemmer_mask(*this, kLastCol, b.getLevel()));
    for (i64 rot = 1; rot < d / 2; rot <<= 1) {
        a.get() = eval_.add(a.get(), eval_.rightRotate(a.get(), rot));
        b.get() = eval_.add(b.get(), eval_.leftRotate(b.get(), rot));
    }
}
// HEMMer::maskFirstRowInplace / maskFirstColOnlyInplace -- HEMMer.cpp:1255-1261, masks :2384-2388, :2418
void HEMMer::maskFirstRowInplace(CtxtTensor &t) { t.get() = eval_.mult(t.get(), hemmer_mask(*this, kFirstRow, t.getLevel())); }
void HEMMer::maskFirstColOnlyInplace(CtxtTensor &t) { t.get() = eval_.mult(t.get(), hemmer_mask(*this, kFirstColOnly, t.getLevel())); }
// HEMMer::maskFirstColInplace / maskLeftHalfInplace / maskRightHalfInplace -- HEMMer.cpp:1251-1269, masks :2378-2394
void HEMMer::maskFirstColInplace(CtxtTensor &t) { t.get() = eval_.mult(t.get(), hemmer_mask(*this, kFirstCol, t.getLevel())); }
void HEMMer::maskLeftHalfInplace(CtxtTensor &t) { t.get() = eval_.mult(t.get(), hemmer_mask(*this, kLeftHalf, t.getLevel())); }
void HEMMer::maskRightHalfInplace(CtxtTensor &t) { t.get() = eval_.mult(t.get(), hemmer_mask(*this, kRightHalf, t.getLevel())); }
// HEMMer::squareSum -- HEMMer.cpp:2499-2510: sum of the tensor squares, one relinearisation and one rescale for the sum
void HEMMer::squareSum(const std::vector<CtxtTensor> &v, CtxtTensor &out) {
    if (v.empty()) throw std::invalid_argument("[squareSum] empty input");
    Ciphertext acc = eval_.tensor(v[0].get(), v[0].get());
    for (size_t i = 1; i < v.size(); ++i) acc = eval_.add(acc, eval_.tensor(v[i].get(), v[i].get()));
    out = CtxtTensor(v[0].getShape(), eval_.rescale(eval_.relinearize(acc)));
}
// HEMMer::reduceRowSumWithScaledMask -- HEMMer.cpp:2512-2530 on one rank: rotate-and-add over a row of the block width,
// the caller's mask (encoded at the ciphertext's level), rotate-and-add back
void HEMMer::reduceRowSumWithScaledMask(CtxtTensor &t, const PtxtTensor &mask) {
    const i64 w = t.getBlockWidth();
    for (i64 i = 1; i < w; i <<= 1) t.get() = eval_.add(t.get(), eval_.leftRotate(t.get(), i));
    t.get() = eval_.mult(t.get(), mask.get());
    for (i64 i = 1; i < w; i <<= 1) t.get() = eval_.add(t.get(), eval_.rightRotate(t.get(), i));
}
// HEMMer::maskRightLeft -- mask_one_left_ / mask_one_right_ of generateRightLeftMasks, HEMMer.cpp:2366-2376
void HEMMer::maskRightLeft(const CtxtTensor &t, CtxtTensor &left, CtxtTensor &right) {
    left = CtxtTensor(t.getShape(), eval_.mult(t.get(), hemmer_mask(*this, kHeadLeft, t.getLevel())));
    right = CtxtTensor(t.getShape(), eval_.mult(t.get(), hemmer_mask(*this, kHeadRight, t.getLevel())));
}
// Gaussian-kernel score assembly -- TransformerBlock.cpp:2420-2482 (one query / key pair; the reference loops over three)
std::vector<CtxtTensor> HEMMer::gaussianKernelScores(const CtxtTensor &query, const CtxtTensor &key, int target_level) {
    std::vector<CtxtTensor> mq(2), mk(2);
    maskRightLeft(query, mq[0], mq[1]);
    maskRightLeft(key, mk[0], mk[1]);
    std::vector<CtxtTensor> oq, ok;
    for (int j = 0; j < 2; ++j) {
        oq.emplace_back(query.getShape(), eval_.square(mq[(size_t)j].get()));
        ok.emplace_back(key.getShape(), eval_.square(mk[(size_t)j].get()));
    }
    oneMatRotSumInplace(oq[0], oq[1]);
    oneMatRotSumInplace(ok[0], ok[1]);
    for (auto &t : ok) transposeInplace(t, target_level);
    std::vector<CtxtTensor> out;
    for (size_t j = 0; j < 2; ++j) {
        complexPackingInplace(mq[j]);
        transposeInplace(mk[j]);
        complexPackingRowInplace(mk[j]);
        CtxtTensor s = repackCC(packedMatMul(mq[j], mk[j], target_level));
        s.get() = eval_.multInteger(s.get(), -2);
        s.get() = eval_.add(s.get(), oq[j].get());
        s.get() = eval_.add(s.get(), ok[j].get());
        out.push_back(std::move(s));
    }
    return out;
}
// the rank-2 LoRA branch of TransformerBlock::attention2_bert_loraOpti -- TransformerBlock.cpp:2199-2365
std::vector<CtxtTensor> HEMMer::loraOptiForward(const std::vector<CtxtTensor> &cur, const CtxtTensor &lora_wa, const CtxtTensor &lora_wb) {
    if (cur.size() != 3) throw std::invalid_argument("[loraOptiForward] three activation pairs expected");
    const i64 d = tile_, w = 2 * tile_;
    // rows 2i and 2i+1 of a factor ciphertext, each moved to row 0, masked and spread over all d rows
    auto rank_rows = [&](const CtxtTensor &factor) {
        std::vector<std::vector<CtxtTensor>> rows;
        for (i64 i = 0; i < 3; ++i) {
            CtxtTensor base = i == 0 ? factor : CtxtTensor(factor.getShape(), eval_.leftRotate(factor.get(), i * 2 * w));
            std::vector<CtxtTensor> pair{base, CtxtTensor(base.getShape(), eval_.leftRotate(base.get(), w))};
            for (auto &t : pair) {
                maskFirstRowInplace(t);
                for (i64 rot = 1; rot < d; rot <<= 1) t.get() = eval_.add(t.get(), eval_.rightRotate(t.get(), rot * w));
            }
            rows.push_back(std::move(pair));
        }
        return rows;
    };
    // X A: slot-wise products summed over the three pairs, then across the 2 d columns of a row into column 0
    const auto wa = rank_rows(lora_wa);
    std::vector<CtxtTensor> xa;
    for (int j = 0; j < 2; ++j) {
        Ciphertext acc = eval_.mult(cur[0].get(), wa[0][(size_t)j].get());
        for (size_t i = 1; i < 3; ++i) acc = eval_.add(acc, eval_.mult(cur[i].get(), wa[i][(size_t)j].get()));
        for (i64 rot = 1; rot < w; rot <<= 1) acc = eval_.add(acc, eval_.leftRotate(acc, rot));
        CtxtTensor t(cur[0].getShape(), std::move(acc));
        maskFirstColOnlyInplace(t);
        xa.push_back(std::move(t));
    }
    // (X A) B: column 0 spread over the row, times the rows of the second factor
    const auto wb = rank_rows(lora_wb);
    for (auto &t : xa)
        for (i64 rot = 1; rot < w; rot <<= 1) t.get() = eval_.add(t.get(), eval_.rightRotate(t.get(), rot));
    std::vector<CtxtTensor> out;
    for (size_t i = 0; i < 3; ++i)
        out.emplace_back(cur[0].getShape(), eval_.add(eval_.mult(xa[0].get(), wb[i][0].get()), eval_.mult(xa[1].get(), wb[i][1].get())));
    return out;
}
// HEMMer::splitInTwo -- HEMMer.cpp:819-831
void HEMMer::splitInTwo(const CtxtTensor &t, CtxtTensor &t1, CtxtTensor &t2) {
    const i64 width = t.getWidth();
    Ciphertext left = eval_.mult(t.get(), hemmer_mask(*this, kLeftHalf, t.getLevel()));
    Ciphertext right = eval_.sub(t.get(), left);
    t1 = CtxtTensor(t.getShape(), eval_.add(eval_.rightRotate(left, width), left));
    t2 = CtxtTensor(t.getShape(), eval_.add(right, eval_.leftRotate(right, width)));
}
// HEMMer::repackCC -- HEMMer.cpp:964-969
CtxtTensor HEMMer::repackCC(const CtxtTensor &t) const { return CtxtTensor(t.getShape(), eval_.add(t.get(), eval_.conjugate(t.get()))); }
// HEMMer::complexPacking(ct, ct) -- HEMMer.cpp:980-986 ; complexPackingRev -- :988-994
CtxtTensor HEMMer::complexPacking(const CtxtTensor &a, const CtxtTensor &b) const { return CtxtTensor(b.getShape(), eval_.add(a.get(), eval_.multImagUnit(b.get()))); }
CtxtTensor HEMMer::complexPackingRev(const CtxtTensor &a, const CtxtTensor &b) const { return CtxtTensor(b.getShape(), eval_.sub(a.get(), eval_.multImagUnit(b.get()))); }
// HEMMer::repack_notBTS -- HEMMer.cpp:1025-1053
CtxtTensor HEMMer::repack_notBTS(const CtxtTensor &t1, const CtxtTensor &t2) {
    Ciphertext a = eval_.rescale(t1.get()), b = eval_.rescale(t2.get());
    Ciphertext out = eval_.add(a, eval_.conjugate(a));
    Ciphertext tmp = eval_.multImagUnit(eval_.add(b, eval_.conjugate(b)));
    out = eval_.add(out, tmp);
    tmp = eval_.leftRotate(out, tile_);
    out = eval_.add(out, tmp);
    tmp = eval_.mult(tmp, hemmer_mask(*this, kLeftHalf, tmp.getLevel()));
    out = eval_.mult(out, hemmer_mask(*this, kLeftHalf, out.getLevel()));
    out = eval_.add(out, eval_.rightRotate(tmp, tile_));
    return CtxtTensor(t1.getShape(), std::move(out));
}
// HEMMer::repack_loraOpti -- HEMMer.cpp:1055-1091; its mask is 0.5 on the left tile (mask_matmul_half_, HEMMer.cpp:2341-2342)
CtxtTensor HEMMer::repack_loraOpti(const CtxtTensor &t1, const CtxtTensor &t2) {
    Ciphertext a = eval_.rescale(t1.get()), b = eval_.rescale(t2.get());
    Ciphertext out = eval_.add(a, eval_.conjugate(a));
    Ciphertext tmp = eval_.multImagUnit(eval_.add(b, eval_.conjugate(b)));
    out = eval_.add(out, tmp);
    tmp = eval_.leftRotate(out, tile_);
    out = eval_.add(out, tmp);
    Ciphertext conj = eval_.conjugate(out);
    out = eval_.add(out, conj);
    tmp = eval_.multImagUnit(eval_.sub(conj, tmp));
    tmp = eval_.mult(tmp, hemmer_mask(*this, kLeftHalfScaled, tmp.getLevel()));
    out = eval_.mult(out, hemmer_mask(*this, kLeftHalfScaled, out.getLevel()));
    out = eval_.add(out, eval_.rightRotate(tmp, tile_));
    return CtxtTensor(t1.getShape(), std::move(out));
}

// ---- LoRA low-rank products and repacking -- HEMMer.cpp:2108-2332 ----
CtxtTensor HEMMer::matMulHighLow(const CtxtTensor &a, const CtxtTensor &b, u64 in_col_block, int t) { HB_ENV; return sched::multMatMatHighLow(env, a, b, (i64)in_col_block, t, low_dim_); }
CtxtTensor HEMMer::matMulLowHigh(const CtxtTensor &a, const CtxtTensor &b, u64 in_row_block, int t) { HB_ENV; return sched::multMatMatLowHigh(env, a, b, (i64)in_row_block, t, low_dim_); }
CtxtTensor HEMMer::matMulLowLow(const CtxtTensor &a, const CtxtTensor &b, u64 in_col_block, u64 in_row_block, int t) {
    HB_ENV; return sched::multMatMatLowLow(env, a, b, (i64)in_col_block, (i64)in_row_block, t, low_dim_);
}
namespace {
enum LowMask { kOneCol = 0, kOneRow, kMultiRow, kColBlock, kRowBlock };
// 0/1 masks that keep one low_dim-wide block: of the first tile only (kOneCol, kOneRow), of every tile across
// the block width (kColBlock, kRowBlock), or a whole row band (kMultiRow)
const Plaintext &low_mask(HEMMer &h, LowMask kind, const TileTensorShape &s, i64 block, int level) {
    const i64 low = h.lowDim();
    MaskCache::Key k{sched::kLowRank, s, ((i64)kind << 40) | (block << 20) | low, level};
    if (const Plaintext *p = h.masks().find(k)) return *p;
    const i64 rows = s.getNumRows(), cols = s.getNumCols(), width = s.getBlockWidth();
    if (rows * width > h.slots() || (block + 1) * low > std::max(rows, width)) throw std::invalid_argument("[lowRank] block outside the tile");
    Message m((size_t)h.slots());
    auto on = [&](i64 r, i64 c) { m.re[(size_t)(r * width + c)] = 1.0; };
    const i64 lo = block * low, hi = (block + 1) * low;
    switch (kind) {
    case kOneCol:   for (i64 r = 0; r < rows; ++r) for (i64 c = lo; c < hi; ++c) on(r, c); break;
    case kOneRow:   for (i64 r = lo; r < hi; ++r) for (i64 c = 0; c < cols; ++c) on(r, c); break;
    case kMultiRow: for (i64 r = lo; r < hi; ++r) for (i64 c = 0; c < width; ++c) on(r, c); break;
    case kColBlock: for (i64 r = 0; r < rows; ++r) for (i64 t = 0; t < width; t += cols) for (i64 c = lo; c < hi; ++c) on(r, t + c); break;
    case kRowBlock: for (i64 r = lo; r < hi; ++r) for (i64 t = 0; t < width; t += cols) for (i64 c = 0; c < cols; ++c) on(r, t + c); break;
    }
    return h.masks().put(k, h.eval().encode(m, level));
}
// x + rot(x, i * step) for i = low, 2 low, ... < end: left when bit j of `pos` is 0, right otherwise.  After the
// tree, block `pos` holds the sum over all blocks.
Ciphertext sum_into_block(const Evaluator &ev, Ciphertext x, i64 low, i64 end, i64 step, i64 pos) {
    for (i64 i = low; i < end; i <<= 1, pos /= 2) x = ev.add(x, pos % 2 == 0 ? ev.leftRotate(x, i * step) : ev.rightRotate(x, i * step));
    return x;
}
}
// HEMMer::repackToOneCol -- HEMMer.cpp:2131-2172
CtxtTensor HEMMer::repackToOneCol(const CtxtTensor &t, u64 out_col_block) {
    const i64 cols = t.getWidth(), width = t.getBlockWidth();
    Ciphertext x = sum_into_block(eval_, t.get(), low_dim_, width, 1, (i64)out_col_block);
    x = eval_.mult(x, low_mask(*this, kOneCol, t.getShape(), (i64)out_col_block, x.getLevel()));
    for (i64 i = cols; i < width; i <<= 1) x = eval_.add(x, eval_.rightRotate(x, cols));
    return CtxtTensor(t.getShape(), std::move(x));
}
// HEMMer::repackToMultiCol -- HEMMer.cpp:2174-2209
CtxtTensor HEMMer::repackToMultiCol(const CtxtTensor &t, u64 out_col_block) {
    Ciphertext x = sum_into_block(eval_, t.get(), low_dim_, t.getBlockWidth() / 2, 1, (i64)out_col_block);
    return CtxtTensor(t.getShape(), eval_.mult(x, low_mask(*this, kColBlock, t.getShape(), (i64)out_col_block, x.getLevel())));
}
// HEMMer::repackToOneRow -- HEMMer.cpp:2211-2255
CtxtTensor HEMMer::repackToOneRow(const CtxtTensor &t, u64 out_row_block) {
    const i64 cols = t.getWidth(), width = t.getBlockWidth();
    Ciphertext x = sum_into_block(eval_, t.get(), low_dim_, t.getHeight(), width, (i64)out_row_block);
    for (i64 i = cols; i < width; i <<= 1) x = eval_.add(x, eval_.leftRotate(x, cols));
    x = eval_.mult(x, low_mask(*this, kOneRow, t.getShape(), (i64)out_row_block, x.getLevel()));
    for (i64 i = cols; i < width; i += cols) x = eval_.add(x, eval_.rightRotate(x, cols));
    return CtxtTensor(t.getShape(), std::move(x));
}
// HEMMer::repackToMultiRow -- HEMMer.cpp:2257-2290
CtxtTensor HEMMer::repackToMultiRow(const CtxtTensor &t, u64 out_row_block) {
    Ciphertext x = sum_into_block(eval_, t.get(), low_dim_, t.getHeight(), t.getBlockWidth(), (i64)out_row_block);
    return CtxtTensor(t.getShape(), eval_.mult(x, low_mask(*this, kMultiRow, t.getShape(), (i64)out_row_block, x.getLevel())));
}
// HEMMer::getLowColBlock -- HEMMer.cpp:2292-2311 ; getLowRowBlock -- :2313-2332
CtxtTensor HEMMer::getLowColBlock(const CtxtTensor &t, u64 col_block) {
    return CtxtTensor(t.getShape(), eval_.mult(t.get(), low_mask(*this, kColBlock, t.getShape(), (i64)col_block, t.getLevel())));
}
CtxtTensor HEMMer::getLowRowBlock(const CtxtTensor &t, u64 row_block) {
    return CtxtTensor(t.getShape(), eval_.mult(t.get(), low_mask(*this, kRowBlock, t.getShape(), (i64)row_block, t.getLevel())));
}

} // namespace HELLM
