// C entry points of libhellm_b200.so: the HEMMer call surface for callers that bind through a C ABI
// (ctypes in this repository's tests and benchmark).  Tile shapes travel as (rows, cols, block_width).
#include "HEMMer.hpp"
#include "hellm_b200.h"

using namespace HELLM;

struct hb_hemmer { hb_ctx *ctx; HEMMer h; explicit hb_hemmer(hb_ctx *c) : ctx(c), h(c) {} };

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
