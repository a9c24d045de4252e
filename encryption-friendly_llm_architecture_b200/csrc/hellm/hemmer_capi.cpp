// C entry points of libhellm_b200.so: the HEMMer call surface for callers that bind through a C ABI
// (ctypes in this repository's tests and benchmark).  Tile shapes travel as (rows, cols, block_width).
#include "HEMMer.hpp"
#include "hellm_b200.h"

using namespace HELLM;

struct hb_hemmer {
    hb_ctx *ctx; HEMMer h; bool owns_ctx = false;
    explicit hb_hemmer(hb_ctx *c) : ctx(c), h(c) {}
    ~hb_hemmer() { h.masks().clear(); if (owns_ctx) hb_ctx_destroy(ctx); }
};

namespace {
// error text for failures raised above the C ABI (the CUDA library keeps its own last-error string)
thread_local std::string g_err;
template <class F> int guard(F &&f) {
    try { f(); return HB_OK; }
    catch (const std::invalid_argument &e) { g_err = e.what(); return HB_E_ARG; }
    catch (const std::exception &e) { g_err = e.what(); return HB_E_CUDA; }
}
// borrow a caller-owned handle for the duration of one call
struct Borrow {
    Ciphertext c;
    Borrow(hb_ctx *ctx, const hb_ct *p) : c(ctx, const_cast<hb_ct *>(p)) {}
    ~Borrow() { c.release(); }
};
CtxtTensor view(Borrow &b, int r, int c, int w) { return CtxtTensor(TileTensorShape(r, c, w), Ciphertext(b.c)); }
}

extern "C" {
const char *hb_hemmer_last_error() { return g_err.c_str(); }
int hb_hemmer_create(hb_ctx *c, hb_hemmer **out) { return guard([&] { *out = new hb_hemmer(c); }); }
void hb_hemmer_destroy(hb_hemmer *h) { delete h; }
// 0 = the reference's rotation sequence (default), 1 = direct, hoisted rotations, 2 = 1 with one division per wrapped copy
int hb_hemmer_set_schedule(hb_hemmer *h, int mode) { if (mode < 0 || mode > 2) return HB_E_ARG; h->h.setSchedule(mode); return HB_OK; }

// HEMMer::genHEMMer (HEMMer.cpp:93-112): context + keys + HEMMer in one call; the object owns the context
int hb_hemmer_gen(int device, const hb_params *prm, hb_hemmer **out) {
    return guard([&] {
        if (!prm || !out) throw std::invalid_argument("[genHEMMer] null argument");
        hb_ctx *c = nullptr;
        if (hb_ctx_create(prm, device, &c) != HB_OK) throw std::runtime_error("[genHEMMer] cannot create a context on this device");
        int rc = hb_keygen(c);
        if (rc != HB_OK) { std::string m = hb_last_error(c); hb_ctx_destroy(c); throw std::runtime_error(m); }
        hb_hemmer *h = new hb_hemmer(c);
        h->owns_ctx = true;
        *out = h;
    });
}
hb_ctx *hb_hemmer_context(const hb_hemmer *h) { return h ? h->ctx : nullptr; }
int hb_hemmer_set_rank(hb_hemmer *h, int rank, int max_rank) { if (!h || rank < 0 || max_rank < 1 || rank >= max_rank) return HB_E_ARG; h->h.setRank(rank, max_rank); return HB_OK; }
int hb_hemmer_get_rank(const hb_hemmer *h) { return h->h.getRank(); }
int hb_hemmer_get_max_rank(const hb_hemmer *h) { return h->h.getMaxRank(); }
int hb_hemmer_save(hb_hemmer *h, const char *keys_path) { return guard([&] { h->h.save(keys_path); }); }

// encode / encrypt / decrypt of row-major matrices (HEMMer.hpp:65-100)
int hb_hemmer_encode(hb_hemmer *h, const double *data, int rows, int cols, int level, hb_pt **out) {
    return guard([&] { *out = h->h.encode(data, rows, cols, level).get().release(); });
}
int hb_hemmer_encode2(hb_hemmer *h, const double *d1, const double *d2, int rows, int cols, int level, hb_pt **out) {
    return guard([&] { *out = h->h.encode2(d1, d2, rows, cols, level).get().release(); });
}
int hb_hemmer_encode_diagonal_to_row4(hb_hemmer *h, const double *w1, const double *w2, const double *w3, const double *w4, int rows, int cols, int level, hb_pt **out) {
    return guard([&] { *out = h->h.encodeDiagonalToRow4(w1, w2, w3, w4, rows, cols, level).get().release(); });
}
int hb_hemmer_encrypt(hb_hemmer *h, const double *data, int rows, int cols, uint64_t nonce, hb_ct **out) {
    return guard([&] { *out = h->h.encrypt(data, rows, cols, nonce).get().release(); });
}
int hb_hemmer_encrypt2(hb_hemmer *h, const double *d1, const double *d2, int rows, int cols, uint64_t nonce, hb_ct **out) {
    return guard([&] { *out = h->h.encrypt2(d1, d2, rows, cols, nonce).get().release(); });
}
int hb_hemmer_decrypt(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, double *out) {
    return guard([&] { Borrow b(h->ctx, a); h->h.decrypt(view(b, rows, cols, width), out); });
}
int hb_hemmer_decrypt2(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, double *out) {
    return guard([&] { Borrow b(h->ctx, a); h->h.decrypt2(view(b, rows, cols, width), out); });
}
int hb_hemmer_add(hb_hemmer *h, const hb_ct *a, const hb_ct *b, hb_ct **out) {
    return guard([&] {
        Borrow ba(h->ctx, a), bb(h->ctx, b);
        CtxtTensor ta(TileTensorShape(), Ciphertext(ba.c));
        h->h.addInplace(ta, CtxtTensor(TileTensorShape(), Ciphertext(bb.c)));
        *out = ta.get().release();
    });
}
int hb_hemmer_hadamard_mult(hb_hemmer *h, const hb_ct *a, const hb_ct *b, hb_ct **out) {
    return guard([&] {
        Borrow ba(h->ctx, a), bb(h->ctx, b);
        CtxtTensor ta(TileTensorShape(), Ciphertext(ba.c));
        h->h.hadamardMultInplace(ta, CtxtTensor(TileTensorShape(), Ciphertext(bb.c)));
        *out = ta.get().release();
    });
}
int hb_hemmer_hadamard_mult_pt(hb_hemmer *h, const hb_ct *a, const hb_pt *p, hb_ct **out) {
    return guard([&] {
        Borrow ba(h->ctx, a);
        CtxtTensor ta(TileTensorShape(), Ciphertext(ba.c));
        h->h.hadamardMultInplace(ta, PtxtTensor(TileTensorShape(), Plaintext::borrowed(p)));
        *out = ta.get().release();
    });
}
int hb_hemmer_one_mat_rot_sum(hb_hemmer *h, const hb_ct *a, const hb_ct *b, hb_ct **out_a, hb_ct **out_b) {
    return guard([&] {
        Borrow ba(h->ctx, a), bb(h->ctx, b);
        CtxtTensor ta(TileTensorShape(), Ciphertext(ba.c)), tb(TileTensorShape(), Ciphertext(bb.c));
        h->h.oneMatRotSumInplace(ta, tb);
        *out_a = ta.get().release(); *out_b = tb.get().release();
    });
}

int hb_hemmer_tr_one_mat_rot_sum(hb_hemmer *h, const hb_ct *a, const hb_ct *b, int target, hb_ct **out_a, hb_ct **out_b) {
    return guard([&] {
        Borrow ba(h->ctx, a), bb(h->ctx, b);
        CtxtTensor ta(TileTensorShape(), Ciphertext(ba.c)), tb(TileTensorShape(), Ciphertext(bb.c));
        h->h.trOneMatRotSumInplace(ta, tb, target);
        *out_a = ta.get().release(); *out_b = tb.get().release();
    });
}

int hb_hemmer_gaussian_kernel_scores(hb_hemmer *h, const hb_ct *query, const hb_ct *key, int rows, int cols, int width, int target, hb_ct **out0, hb_ct **out1) {
    return guard([&] {
        Borrow bq(h->ctx, query), bk(h->ctx, key);
        std::vector<CtxtTensor> r = h->h.gaussianKernelScores(view(bq, rows, cols, width), view(bk, rows, cols, width), target);
        *out0 = r[0].get().release(); *out1 = r[1].get().release();
    });
}
int hb_hemmer_lora_opti_forward(hb_hemmer *h, const hb_ct *cur0, const hb_ct *cur1, const hb_ct *cur2, const hb_ct *lora_wa, const hb_ct *lora_wb, hb_ct **out0,
                                hb_ct **out1, hb_ct **out2) {
    return guard([&] {
        Borrow b0(h->ctx, cur0), b1(h->ctx, cur1), b2(h->ctx, cur2), ba(h->ctx, lora_wa), bb(h->ctx, lora_wb);
        const i64 d = h->h.tile();
        const TileTensorShape s(d, d, 2 * d);
        std::vector<CtxtTensor> cur{CtxtTensor(s, Ciphertext(b0.c)), CtxtTensor(s, Ciphertext(b1.c)), CtxtTensor(s, Ciphertext(b2.c))};
        std::vector<CtxtTensor> r = h->h.loraOptiForward(cur, CtxtTensor(s, Ciphertext(ba.c)), CtxtTensor(s, Ciphertext(bb.c)));
        *out0 = r[0].get().release(); *out1 = r[1].get().release(); *out2 = r[2].get().release();
    });
}

#define SHAPE_ARGS int rows, int cols, int width
#define IN_TENSOR(name, p) Borrow name##_b(h->ctx, p); CtxtTensor name(TileTensorShape(rows, cols, width), Ciphertext(name##_b.c))

int hb_hemmer_transpose(hb_hemmer *h, const hb_ct *a, SHAPE_ARGS, int target, hb_ct **out) {
    return guard([&] { IN_TENSOR(t, a); h->h.transposeInplace(t, target); *out = t.get().release(); });
}
int hb_hemmer_sigma(hb_hemmer *h, const hb_ct *a, SHAPE_ARGS, hb_ct **out) {
    return guard([&] { IN_TENSOR(t, a); *out = h->h.diagonalToColumn(t).get().release(); });
}
int hb_hemmer_tau(hb_hemmer *h, const hb_ct *a, SHAPE_ARGS, hb_ct **out) {
    return guard([&] { IN_TENSOR(t, a); *out = h->h.diagonalToRow(t).get().release(); });
}
int hb_hemmer_mask_inplace(hb_hemmer *h, const hb_ct *a, int which, SHAPE_ARGS, hb_ct **out) {
    return guard([&] {
        IN_TENSOR(t, a);
        if (which == 0) h->h.maskFirstColInplace(t);
        else if (which == 1) h->h.maskLeftHalfInplace(t);
        else if (which == 2) h->h.maskRightHalfInplace(t);
        else throw std::invalid_argument("[mask] unknown mask");
        *out = t.get().release();
    });
}
int hb_hemmer_square_sum(hb_hemmer *h, const hb_ct *const *v, int count, SHAPE_ARGS, hb_ct **out) {
    return guard([&] {
        std::vector<std::unique_ptr<Borrow>> hold;
        std::vector<CtxtTensor> ts;
        for (int i = 0; i < count; ++i) { hold.emplace_back(new Borrow(h->ctx, v[i])); ts.push_back(view(*hold.back(), rows, cols, width)); }
        CtxtTensor o;
        h->h.squareSum(ts, o);
        *out = o.get().release();
    });
}
int hb_hemmer_reduce_row_sum_with_scaled_mask(hb_hemmer *h, const hb_ct *a, const hb_pt *mask, SHAPE_ARGS, hb_ct **out) {
    return guard([&] {
        IN_TENSOR(t, a);
        PtxtTensor m(TileTensorShape(rows, cols, width), Plaintext::borrowed(mask));
        h->h.reduceRowSumWithScaledMask(t, m);
        *out = t.get().release();
    });
}
int hb_hemmer_matmul_cc(hb_hemmer *h, const hb_ct *a, int ra, int ca, int wa, const hb_ct *b, int rb, int cb, int wb, int target, hb_ct **out) {
    return guard([&] {
        Borrow ba(h->ctx, a), bb(h->ctx, b);
        CtxtTensor ta = view(ba, ra, ca, wa), tb = view(bb, rb, cb, wb);
        *out = h->h.singleCCMatMul(ta, tb, target).get().release();
    });
}
int hb_hemmer_matmul_cp(hb_hemmer *h, const hb_ct *a, int ra, int ca, int wa, const hb_pt *b, int rb, int cb, int wb, int target, hb_ct **out) {
    return guard([&] {
        Borrow ba(h->ctx, a);
        CtxtTensor ta = view(ba, ra, ca, wa);
        PtxtTensor tb(TileTensorShape(rb, cb, wb), Plaintext::borrowed(b));
        *out = h->h.singleMatMul(ta, tb, target).get().release();
    });
}
int hb_hemmer_matmul_cc_prepare(hb_hemmer *h, const hb_ct *a, int ra, int ca, int wa, const hb_ct *b, int rb, int cb, int wb, int target, hb_ct **out_a, hb_ct **out_b) {
    return guard([&] {
        Borrow ba(h->ctx, a), bb(h->ctx, b);
        CtxtTensor ta = view(ba, ra, ca, wa), tb = view(bb, rb, cb, wb);
        Ciphertext sa, sb;
        h->h.ccMatMulPrepare(ta, tb, target, sa, sb);
        *out_a = sa.release(); *out_b = sb.release();
    });
}
int hb_hemmer_matmul_cc_core(hb_hemmer *h, const hb_ct *sa, const hb_ct *tb, int rows, int inner, int cols, int width, int target, hb_ct **out) {
    return guard([&] {
        Borrow ba(h->ctx, sa), bb(h->ctx, tb);
        *out = h->h.ccMatMulCore(Ciphertext(ba.c), Ciphertext(bb.c), rows, inner, cols, width, target).get().release();
    });
}
int hb_hemmer_packed_matmul(hb_hemmer *h, const hb_ct *a, int ra, int ca, int wa, const hb_ct *b, int rb, int cb, int wb, int target, hb_ct **out) {
    return guard([&] {
        Borrow ba(h->ctx, a), bb(h->ctx, b);
        CtxtTensor ta = view(ba, ra, ca, wa), tb = view(bb, rb, cb, wb);
        *out = h->h.packedMatMul(ta, tb, target).get().release();
    });
}
int hb_hemmer_matmul_pre(hb_hemmer *h, const hb_ct *a, SHAPE_ARGS, int target, hb_ct **out) {
    return guard([&] { IN_TENSOR(t, a); *out = h->h.matMulPre(t, target).release(); });
}
int hb_hemmer_matmul_reuse(hb_hemmer *h, const hb_ct *pre, const hb_pt *p, SHAPE_ARGS, hb_ct **out) {
    return guard([&] {
        Borrow bp(h->ctx, pre);
        // the plaintext stays owned by the caller: wrap it without a deleter
        hb_ct *o = nullptr;
        int lp = 0, lc = 0; hb_pt_meta(p, &lp, nullptr); hb_ct_meta(pre, &lc, nullptr, nullptr, nullptr);
        if (lp != lc) throw std::invalid_argument("[multMatMatReUse] plaintext level differs from the ciphertexts'");
        check(h->ctx, hb_matmul_acc(h->ctx, pre, p, width, &o));
        (void)rows; (void)cols;
        *out = o;
    });
}
// matMulReUse summed over K-groups: pre holds the copies of `btotal` inputs, groups b0..b0+bcount-1 meet pts[0..bcount-1]
int hb_hemmer_matmul_reuse_groups(hb_hemmer *h, const hb_ct *pre, int btotal, int b0, const hb_pt *const *pts, int bcount, int width, hb_ct **out) {
    return guard([&] { hb_ct *o = nullptr; check(h->ctx, hb_matmul_acc_multi(h->ctx, pre, btotal, b0, pts, bcount, width, &o)); *out = o; });
}
int hb_hemmer_matmul_reuse_groups_tiles(hb_hemmer *h, const hb_ct *pre, int btotal, int b0, const hb_pt *const *pts, int bcount, int tiles, int width, hb_ct **out) {
    return guard([&] { check(h->ctx, hb_matmul_acc_tiles(h->ctx, pre, btotal, b0, pts, bcount, tiles, width, out)); });
}
int hb_hemmer_matmul_pre_rev(hb_hemmer *h, const hb_ct *b, SHAPE_ARGS, int target, hb_ct **out) {
    return guard([&] { IN_TENSOR(t, b); *out = h->h.matMulPreRev(t, target).get().release(); });
}
int hb_hemmer_matmul_cc_reuse(hb_hemmer *h, const hb_ct *pre, const hb_ct *b, SHAPE_ARGS, hb_ct **out) {
    return guard([&] { Borrow bp(h->ctx, pre); IN_TENSOR(t, b); *out = h->h.matMulCCReUse(bp.c, t).get().release(); });
}
int hb_hemmer_packed_matmul_pre(hb_hemmer *h, const hb_ct *a, SHAPE_ARGS, int target, hb_ct **out) {
    return guard([&] { IN_TENSOR(t, a); *out = h->h.packedMatMulPre(t, target).get().release(); });
}
int hb_hemmer_packed_matmul_pre_rot(hb_hemmer *h, const hb_ct *a, SHAPE_ARGS, int target, hb_ct **out) {
    return guard([&] { IN_TENSOR(t, a); *out = h->h.packedMatMulPreRot(t, target).release(); });
}
int hb_hemmer_packed_matmul_pre_rev(hb_hemmer *h, const hb_ct *b, SHAPE_ARGS, int target, hb_ct **out) {
    return guard([&] { IN_TENSOR(t, b); *out = h->h.packedMatMulPreRev(t, target).get().release(); });
}
int hb_hemmer_packed_matmul_cc_reuse(hb_hemmer *h, const hb_ct *pre, const hb_ct *b, SHAPE_ARGS, hb_ct **out) {
    return guard([&] { Borrow bp(h->ctx, pre); IN_TENSOR(t, b); *out = h->h.packedMatMulCCReuse(bp.c, t).get().release(); });
}
int hb_hemmer_complex_packing(hb_hemmer *h, const hb_ct *a, SHAPE_ARGS, hb_ct **out) {
    return guard([&] { IN_TENSOR(t, a); h->h.complexPackingInplace(t); *out = t.get().release(); });
}
int hb_hemmer_complex_packing_row(hb_hemmer *h, const hb_ct *a, SHAPE_ARGS, hb_ct **out) {
    return guard([&] { IN_TENSOR(t, a); h->h.complexPackingRowInplace(t); *out = t.get().release(); });
}
int hb_hemmer_transpose_complex_packing(hb_hemmer *h, const hb_ct *a, SHAPE_ARGS, int target, hb_ct **out) {
    return guard([&] { IN_TENSOR(t, a); h->h.transposeComplexPackingInplace(t, target); *out = t.get().release(); });
}
int hb_hemmer_split_in_two(hb_hemmer *h, const hb_ct *a, SHAPE_ARGS, hb_ct **out1, hb_ct **out2) {
    return guard([&] { IN_TENSOR(t, a); CtxtTensor t1, t2; h->h.splitInTwo(t, t1, t2); *out1 = t1.get().release(); *out2 = t2.get().release(); });
}
int hb_hemmer_repack_cc(hb_hemmer *h, const hb_ct *a, hb_ct **out) {
    return guard([&] { Borrow ba(h->ctx, a); *out = h->h.repackCC(CtxtTensor(TileTensorShape(), Ciphertext(ba.c))).get().release(); });
}
int hb_hemmer_complex_packing2(hb_hemmer *h, const hb_ct *a, const hb_ct *b, hb_ct **out) {
    return guard([&] {
        Borrow ba(h->ctx, a), bb(h->ctx, b);
        *out = h->h.complexPacking(CtxtTensor(TileTensorShape(), Ciphertext(ba.c)), CtxtTensor(TileTensorShape(), Ciphertext(bb.c))).get().release();
    });
}
int hb_hemmer_complex_packing_rev(hb_hemmer *h, const hb_ct *a, const hb_ct *b, hb_ct **out) {
    return guard([&] {
        Borrow ba(h->ctx, a), bb(h->ctx, b);
        *out = h->h.complexPackingRev(CtxtTensor(TileTensorShape(), Ciphertext(ba.c)), CtxtTensor(TileTensorShape(), Ciphertext(bb.c))).get().release();
    });
}
int hb_hemmer_repack_not_bts(hb_hemmer *h, const hb_ct *a, const hb_ct *b, hb_ct **out) {
    return guard([&] {
        Borrow ba(h->ctx, a), bb(h->ctx, b);
        *out = h->h.repack_notBTS(CtxtTensor(TileTensorShape(), Ciphertext(ba.c)), CtxtTensor(TileTensorShape(), Ciphertext(bb.c))).get().release();
    });
}
int hb_hemmer_repack_lora_opti(hb_hemmer *h, const hb_ct *a, const hb_ct *b, hb_ct **out) {
    return guard([&] {
        Borrow ba(h->ctx, a), bb(h->ctx, b);
        *out = h->h.repack_loraOpti(CtxtTensor(TileTensorShape(), Ciphertext(ba.c)), CtxtTensor(TileTensorShape(), Ciphertext(bb.c))).get().release();
    });
}
// LoRA low-rank family (HEMMer.cpp:2108-2332); low_dim replaces the compile-time ModelArgs::LOW_DIM
int hb_hemmer_matmul_high_low(hb_hemmer *h, const hb_ct *a, int ra, int ca, int wa, const hb_ct *b, int rb, int cb, int wb, int in_col_block, int target, int low_dim, hb_ct **out) {
    return guard([&] {
        Borrow ba(h->ctx, a), bb(h->ctx, b);
        h->h.setLowDim(low_dim);
        *out = h->h.matMulHighLow(view(ba, ra, ca, wa), view(bb, rb, cb, wb), (u64)in_col_block, target).get().release();
    });
}
int hb_hemmer_matmul_low_high(hb_hemmer *h, const hb_ct *a, int ra, int ca, int wa, const hb_ct *b, int rb, int cb, int wb, int in_row_block, int target, int low_dim, hb_ct **out) {
    return guard([&] {
        Borrow ba(h->ctx, a), bb(h->ctx, b);
        h->h.setLowDim(low_dim);
        *out = h->h.matMulLowHigh(view(ba, ra, ca, wa), view(bb, rb, cb, wb), (u64)in_row_block, target).get().release();
    });
}
int hb_hemmer_matmul_low_low(hb_hemmer *h, const hb_ct *a, int ra, int ca, int wa, const hb_ct *b, int rb, int cb, int wb, int in_col_block, int in_row_block, int target, int low_dim, hb_ct **out) {
    return guard([&] {
        Borrow ba(h->ctx, a), bb(h->ctx, b);
        h->h.setLowDim(low_dim);
        *out = h->h.matMulLowLow(view(ba, ra, ca, wa), view(bb, rb, cb, wb), (u64)in_col_block, (u64)in_row_block, target).get().release();
    });
}
#define LOW_REPACK(name, method) \
    int hb_hemmer_##name(hb_hemmer *h, const hb_ct *a, SHAPE_ARGS, int block, int low_dim, hb_ct **out) { \
        return guard([&] { if (block < 0) throw std::invalid_argument("[lowRank] negative block"); IN_TENSOR(t, a); h->h.setLowDim(low_dim); *out = h->h.method(t, (u64)block).get().release(); }); \
    }
LOW_REPACK(repack_to_one_col, repackToOneCol)
LOW_REPACK(repack_to_multi_col, repackToMultiCol)
LOW_REPACK(repack_to_one_row, repackToOneRow)
LOW_REPACK(repack_to_multi_row, repackToMultiRow)
LOW_REPACK(low_col_block, getLowColBlock)
LOW_REPACK(low_row_block, getLowRowBlock)
} // extern "C"
