// Diagonal / rotate-and-accumulate schedules for encrypted tile products.
//
// Algorithm (Jiang-Kim-Lauter-Song style, as scheduled by the reference in
// ciphertext/src/MatrixUtils.cpp): with sigma(A)[r][c] = A[r][c+r] and tau(B)[r][c] = B[r+c][c],
//     A*B = sum_k  phi^k(sigma A) (.) psi^k(tau B),
// phi^k a column shift with wrap inside the row, psi^k a row shift.  sigma, tau and the transpose
// are sums of masked rotations arranged as baby-step / giant-step.  The ciphertext bits depend on
// the order of operations, so each function keeps the order of the reference function it names;
// what differs is that masks are encoded once per level and kept on the device, and that the
// mask-mask-add-rescale "assemble" step and the tensor accumulation are single fused launches.
#include "schedules.hpp"

#include <cmath>
#include <functional>

namespace HELLM {
namespace sched {

namespace {

i64 ceil_pow2(i64 v) { i64 p = 1; while (p < v) p <<= 1; return p; }
i64 ceil_sqrt(i64 v) { return (i64)std::ceil(std::sqrt((double)v)); }
i64 ceil_div(i64 a, i64 b) { return (i64)std::ceil((double)a / (double)b); }

// ---- mask construction -------------------------------------------------------------------
// A mask is a 0/value indicator over (row, col) of one tile, copied to a set of tile origins in
// the slot grid, then pre-rotated by the amount the giant step will undo.
using Pred = std::function<bool(i64 row, i64 col)>;

struct Placement { std::vector<std::pair<i64, i64>> origins; i64 row_scale = 1, col_scale = 1; };

Placement all_blocks(const Env &e, const TileTensorShape &s) { // every rows x cols block of the grid
    Placement p;
    const i64 height = e.slots / s.getBlockWidth();
    for (i64 rb = 0; rb < height; rb += s.getNumRows())
        for (i64 cb = 0; cb < s.getBlockWidth(); cb += s.getNumCols()) p.origins.push_back({rb, cb});
    return p;
}
Message paint(const Env &e, const TileTensorShape &s, const Placement &pl, i64 rows, i64 cols, const Pred &pred, double value) {
    Message m((size_t)e.slots);
    const i64 w = s.getBlockWidth();
    for (i64 r = 0; r < rows; ++r)
        for (i64 c = 0; c < cols; ++c) {
            if (!pred(r, c)) continue;
            for (const auto &o : pl.origins)
                for (i64 dr = 0; dr < pl.row_scale; ++dr)
                    for (i64 dc = 0; dc < pl.col_scale; ++dc)
                        m.re[(size_t)((o.first + pl.row_scale * r + dr) * w + o.second + pl.col_scale * c + dc)] = value;
        }
    return m;
}

const Plaintext &cached(Env &e, int kind, const TileTensorShape &s, i64 idx, int level, const std::function<Message()> &make, bool extended = false) {
    MaskCache::Key k{kind, s, idx, level};
    if (const Plaintext *p = e.cache.find(k)) return *p;
    return e.cache.put(k, extended ? e.ev.encodeExtended(make(), level) : e.ev.encode(make(), level));
}

// Masks of sigma / tau and their packed forms.
//   horizontal (MatrixUtils.cpp:129-217): idx = 0 keeps rows = 0 (mod sub); idx > 0 keeps rows = idx (mod sub),
//   columns < cols - idx; idx < 0 keeps rows = cols + idx (mod sub), columns >= -idx.  The vertical family
//   (:330-419) is the same with rows and columns exchanged.  Each mask is rotated by the amount its giant step
//   undoes.  Packed families (:219-328, :421-527) work on the grid of 2x2 slot blocks; the horizontal one
//   carries 1/2, and both are painted on the two tiles of a side-by-side pair only.
struct DiagFamily {
    bool vertical, packed;
    i64 rows, cols, sub, main, bs, gs, gap;
};
DiagFamily family(const TileTensorShape &s, bool vertical, bool packed) {
    DiagFamily f{};
    f.vertical = vertical; f.packed = packed;
    f.rows = packed ? s.getNumRows() / 2 : s.getNumRows();
    f.cols = packed ? s.getNumCols() / 2 : s.getNumCols();
    f.sub = std::min(f.rows, f.cols);
    f.main = vertical ? f.rows : f.cols;
    f.bs = ceil_sqrt(2 * f.sub - 1);
    f.gs = ceil_div(f.sub - 1, f.bs);
    const i64 unit = vertical ? s.getBlockWidth() : 1;
    f.gap = packed ? 2 * unit : unit;
    return f;
}
Message diag_family_mask(const Env &e, const TileTensorShape &s, const DiagFamily &f, i64 idx) {
    const i64 sub = f.sub, main = f.main;
    Pred pred;
    if (idx == 0) pred = [=](i64 r, i64 c) { return ((f.vertical ? c : r) % sub) == 0; };
    else if (idx > 0) pred = [=](i64 r, i64 c) { i64 a = f.vertical ? c : r, b = f.vertical ? r : c; return a >= idx && (a - idx) % sub == 0 && b < main - idx; };
    else pred = [=](i64 r, i64 c) { i64 a = f.vertical ? c : r, b = f.vertical ? r : c; return a >= main + idx && (a - main - idx) % sub == 0 && b >= -idx; };
    Placement pl;
    if (f.packed) {
        pl.row_scale = pl.col_scale = 2;
        pl.origins.push_back({0, 0});
        if (s.getBlockWidth() != f.cols) pl.origins.push_back({0, 2 * f.cols});
    } else {
        pl = all_blocks(e, s);
    }
    Message m = paint(e, s, pl, f.rows, f.cols, pred, (f.packed && !f.vertical) ? 0.5 : 1.0);
    if (idx == 0) return m;
    // giant-step index this mask belongs to, and the rotation applied after the baby-step sum
    const i64 i = idx > 0 ? (idx - 1) / f.bs : (idx + main - 1) / f.bs;
    const i64 rot_num = i * f.bs * f.gap;
    return m.rotated_right(idx > 0 ? rot_num : rot_num - main * f.gap);
}

// Baby-step / giant-step evaluation shared by diagonalToColumn (MatrixUtils.cpp:776-848), diagonalToRow
// (:924-996), packedDiagonalToColumn (:850-922) and packedDiagonalToRow (:998-1070).
Ciphertext bsgs_diagonals(Env &e, const Ciphertext &op, const TileTensorShape &s, bool vertical, bool packed) {
    const DiagFamily f = family(s, vertical, packed);
    const int kind = packed ? (vertical ? kPackedVertical : kPackedHorizontal) : (vertical ? kVertical : kHorizontal);
    const int level = op.getLevel();
    auto mask = [&](i64 idx) -> const Plaintext & { return cached(e, kind, s, idx, level, [&] { return diag_family_mask(e, s, f, idx); }); };
    std::vector<Ciphertext> baby;
    baby.reserve((size_t)f.bs);
    if (e.mode >= kDirect) {
        const Hoisted h = e.ev.decompose(op);
        for (i64 j = 0; j < f.bs; ++j) baby.push_back(e.ev.leftRotate(op, h, (j + 1) * f.gap));
    } else {
        baby.push_back(e.ev.leftRotate(op, f.gap));
        for (i64 j = 1; j < f.bs; ++j) baby.push_back(e.ev.leftRotate(baby.back(), f.gap));
    }
    // kLazy: the parts and their giant steps are collected and rotated by ONE call that shares the ModDown; when they
    // fit its limits, all parts are also formed by one pass over the baby steps (terms: op, baby[0], baby[1], ...)
    if (e.mode == kLazy && (size_t)f.bs + 1 <= Evaluator::kMaxPartTerms && (size_t)(2 * f.gs + 1) <= Evaluator::kMaxParts) {
        std::vector<const Ciphertext *> terms{&op};
        for (i64 j = 0; j < f.bs; ++j) terms.push_back(&baby[(size_t)j]);
        std::vector<std::vector<const Plaintext *>> rows;
        std::vector<i64> steps;
        rows.push_back({&mask(0)}); steps.push_back(0);
        for (i64 i = 0; i < f.gs; ++i) {
            const i64 rot_num = i * f.bs * f.gap;
            for (int sign = -1; sign <= 1; sign += 2) {
                i64 idx = 1 + i * f.bs + (sign < 0 ? -f.main : 0);
                const i64 limit = sign < 0 ? f.sub - f.main : f.sub;
                std::vector<const Plaintext *> row(terms.size(), nullptr);
                row[1] = &mask(idx);
                for (i64 j = 1; j < f.bs; ++j) {
                    if (++idx >= limit) break;
                    row[(size_t)j + 1] = &mask(idx);
                }
                rows.push_back(std::move(row));
                steps.push_back(sign < 0 ? -(f.main * f.gap - rot_num) : rot_num);
            }
        }
        return e.ev.rotateSumGrouped(e.ev.multSumRescaledOnceParts(terms, rows), steps);
    }
    std::vector<Ciphertext> parts; std::vector<i64> part_steps;
    Ciphertext res = e.ev.mult(op, mask(0));
    if (e.mode == kLazy) { parts.push_back(std::move(res)); part_steps.push_back(0); }
    for (i64 i = 0; i < f.gs; ++i) {
        const i64 rot_num = i * f.bs * f.gap;
        for (int sign = -1; sign <= 1; sign += 2) { // negative diagonals first, then positive
            i64 idx = 1 + i * f.bs + (sign < 0 ? -f.main : 0);
            const i64 limit = sign < 0 ? f.sub - f.main : f.sub;
            // baby-step sum: part = sum_j mult(baby[j], mask[idx + j]), one fused call
            std::vector<const Ciphertext *> cts{&baby[0]};
            std::vector<const Plaintext *> pts{&mask(idx)};
            for (i64 j = 1; j < f.bs; ++j) {
                if (++idx >= limit) break;
                cts.push_back(&baby[(size_t)j]); pts.push_back(&mask(idx));
            }
            if (e.mode == kLazy) {
                parts.push_back(e.ev.multSumRescaledOnce(cts, pts));
                part_steps.push_back(sign < 0 ? -(f.main * f.gap - rot_num) : rot_num);
                continue;
            }
            Ciphertext part = e.ev.multSum(cts, pts);
            part = sign < 0 ? e.ev.rightRotate(part, f.main * f.gap - rot_num) : e.ev.leftRotate(part, rot_num);
            res = e.ev.add(res, part);
        }
    }
    if (e.mode == kLazy) return e.ev.rotateSum(parts, part_steps);
    return res;
}

// Column / row wrap masks of the shift loops (generateColMask / generateRowMask, MatrixUtils.cpp:529-578):
// entry 2i is 1 where the shifted copy has wrapped (last i columns / rows), entry 2i+1 its complement.  They are
// encoded with the extra special-prime limbs so that the kLazy schedule can apply them to a key-switch result that
// is still in the extended basis; the first level + 1 limbs are those of a plain encoding.
const Plaintext &col_wrap(Env &e, const TileTensorShape &s, i64 which, int level) {
    return cached(e, kColWrap, s, which, level, [&] {
        Message m((size_t)e.slots);
        const i64 cols = s.getNumCols(), i = which / 2; const bool wrapped = (which % 2) == 0;
        for (i64 j = 0; j < e.slots; ++j) { bool in_tail = (j % cols) >= cols - i; m.re[(size_t)j] = (in_tail == wrapped) ? 1.0 : 0.0; }
        return m;
    }, true);
}
const Plaintext &row_wrap(Env &e, const TileTensorShape &s, i64 which, int level) {
    return cached(e, kRowWrap, s, which, level, [&] {
        Message m((size_t)e.slots);
        const i64 rows = s.getNumRows(), w = s.getBlockWidth(), i = which / 2; const bool wrapped = (which % 2) == 0;
        for (i64 j = 0; j < e.slots; ++j) { bool in_tail = ((j / w) % rows) >= rows - i; m.re[(size_t)j] = (in_tail == wrapped) ? 1.0 : 0.0; }
        return m;
    }, true);
}

// The wrapped copy number i of a shift loop, rescale(wrap[2i+1] (.) rot(x, s) + wrap[2i] (.) rot(x, s_wrapped)), in the kLazy
// schedule: the two masks are folded into their rotation keys once (cached per shape, shift and level).  When both
// steps are the same rotation (a row shift by the whole tile height on a full slot grid) one key carries both masks.
struct WrappedCopy { const MaskedKey *main; const MaskedKey *wrapped; };
WrappedCopy wrapped_copy(Env &e, bool rows, const TileTensorShape &s, i64 i, int level, i64 step, i64 step_wrapped) {
    const int kind = rows ? kRowWrapKey : kColWrapKey;
    const i64 norm = e.slots;
    const bool same = ((step - step_wrapped) % norm) == 0;
    // the steps are part of the key: the wrapped step depends on the other operand's width as well as on the shape
    const i64 st = ((step % norm) + norm) % norm, sw = ((step_wrapped % norm) + norm) % norm, tag = (st << 20) | (sw << 40);
    MaskCache::Key k1{kind, s, tag | (2 * i + 1), level}, k0{kind, s, tag | (2 * i), level};
    const MaskedKey *main = e.cache.findKey(k1);
    if (!main) {
        const Plaintext &m1 = rows ? row_wrap(e, s, 2 * i + 1, level) : col_wrap(e, s, 2 * i + 1, level);
        const Plaintext &m0 = rows ? row_wrap(e, s, 2 * i, level) : col_wrap(e, s, 2 * i, level);
        main = &e.cache.putKey(k1, same ? e.ev.maskedKey(step, m1, &m0) : e.ev.maskedKey(step, m1));
        if (!same) e.cache.putKey(k0, e.ev.maskedKey(step_wrapped, m0));
    }
    return WrappedCopy{main, same ? nullptr : e.cache.findKey(k0)};
}
// Wrapped copies first .. first + count - 1 of one operand in one launch sequence (group-major batch).
Ciphertext assemble_lazy(Env &e, const Ciphertext &x, const Hoisted &h, const std::vector<WrappedCopy> &w) {
    std::vector<const MaskedKey *> ka, kb;
    for (const auto &c : w) { ka.push_back(c.main); kb.push_back(c.wrapped); }
    return e.ev.assembleRotationsMulti(x, h, ka, kb);
}
// Iterations of a shift loop handled by one launch sequence: batches are stacked until about 168 ciphertexts are in
// flight.  A batch of 40 fills the GPU on its own; beyond that the gain is the accumulator of the product loop, which is
// read and written once per launch sequence instead of once per iteration.  The stored residues do not depend on the grouping.
i64 loop_group(const Ciphertext &x) { return std::max<i64>(1, std::min<i64>(16, 168 / std::max(1, x.getBatch()))); }

void require_product_shapes(const CtxtTensor &a, const CtxtTensor &b) {
    if (a.getWidth() != b.getHeight()) throw std::invalid_argument("[getCommonInsideLength] different inside length.");
    if (a.getBlockWidth() != b.getBlockWidth()) throw std::invalid_argument("[getCommonBlockWidth] different block width");
}

} // namespace

// MatrixTransformer::transpose<Ciphertext> -- MatrixUtils.cpp:671-739, masks :90-127.
// Diagonal delta = col - row of the result moves by (width-1)*delta slots.
CtxtTensor transpose(Env &e, const CtxtTensor &op) {
    const i64 num_cols = op.getHeight(), num_rows = op.getWidth(), width = op.getBlockWidth();
    if (num_cols > width) throw std::invalid_argument("[transpose] num_cols > width.");
    const TileTensorShape s(num_rows, num_cols, width);
    const i64 count = num_rows + num_cols - 1, bs = ceil_sqrt(count), gs = ceil_div(count, bs), gap = width - 1;
    const int level = op.get().getLevel();
    auto mask = [&](i64 idx) -> const Plaintext & {
        return cached(e, kDiagonal, s, idx, level, [&] {
            Placement pl; pl.origins.push_back({0, 0});
            if (width != num_cols) pl.origins.push_back({0, num_rows});
            Message m = paint(e, s, pl, num_rows, num_cols, [=](i64 r, i64 c) { return c - r == idx; }, 1.0);
            const i64 i = (idx - (1 - num_rows)) / bs;
            return m.rotated_right(i * bs * gap);
        });
    };
    std::vector<Ciphertext> baby;
    baby.reserve((size_t)bs);
    if (e.mode >= kDirect) {
        const Hoisted h = e.ev.decompose(op.get());
        for (i64 j = 0; j < bs; ++j) baby.push_back(e.ev.leftRotate(op.get(), h, (j - (num_rows - 1)) * gap));
    } else {
        baby.push_back(e.ev.rightRotate(op.get(), (num_rows - 1) * gap));
        for (i64 j = 1; j < bs; ++j) baby.push_back(e.ev.leftRotate(baby.back(), gap));
    }
    Ciphertext res;
    if (e.mode == kLazy && (size_t)bs <= Evaluator::kMaxPartTerms && (size_t)gs <= Evaluator::kMaxParts) { // all parts by one pass over the baby steps
        std::vector<const Ciphertext *> terms;
        for (i64 j = 0; j < bs; ++j) terms.push_back(&baby[(size_t)j]);
        std::vector<std::vector<const Plaintext *>> rows;
        std::vector<i64> steps;
        for (i64 i = 0; i < gs; ++i) {
            i64 idx = 1 - num_rows + i * bs;
            std::vector<const Plaintext *> row(terms.size(), nullptr);
            row[0] = &mask(idx);
            for (i64 j = 1; j < bs; ++j) {
                if (++idx >= num_cols) break;
                row[(size_t)j] = &mask(idx);
            }
            rows.push_back(std::move(row));
            steps.push_back(i * bs * gap);
        }
        return CtxtTensor(s, e.ev.rotateSumGrouped(e.ev.multSumRescaledOnceParts(terms, rows), steps));
    }
    std::vector<Ciphertext> parts; std::vector<i64> part_steps; // kLazy: all giant steps in one call
    for (i64 i = 0; i < gs; ++i) {
        i64 idx = 1 - num_rows + i * bs;
        std::vector<const Ciphertext *> cts{&baby[0]};
        std::vector<const Plaintext *> pts{&mask(idx)};
        for (i64 j = 1; j < bs; ++j) {
            if (++idx >= num_cols) break;
            cts.push_back(&baby[(size_t)j]); pts.push_back(&mask(idx));
        }
        if (e.mode == kLazy) { parts.push_back(e.ev.multSumRescaledOnce(cts, pts)); part_steps.push_back(i * bs * gap); continue; }
        Ciphertext part = e.ev.multSum(cts, pts);
        if (i == 0) res = std::move(part);
        else res = e.ev.add(res, e.ev.leftRotate(part, i * bs * gap));
    }
    if (e.mode == kLazy) res = e.ev.rotateSum(parts, part_steps);
    return CtxtTensor(s, std::move(res));
}

CtxtTensor diagonalToColumn(Env &e, const CtxtTensor &op) { return CtxtTensor(op.getShape(), bsgs_diagonals(e, op.get(), op.getShape(), false, false)); }
CtxtTensor diagonalToRow(Env &e, const CtxtTensor &op) { return CtxtTensor(op.getShape(), bsgs_diagonals(e, op.get(), op.getShape(), true, false)); }
CtxtTensor packedDiagonalToColumn(Env &e, const CtxtTensor &op) {
    const TileTensorShape s(2 * (op.getHeight() / 2), 2 * (op.getWidth() / 2), op.getBlockWidth());
    return CtxtTensor(s, bsgs_diagonals(e, op.get(), s, false, true));
}
CtxtTensor packedDiagonalToRow(Env &e, const CtxtTensor &op) {
    const TileTensorShape s(2 * (op.getHeight() / 2), 2 * (op.getWidth() / 2), op.getBlockWidth());
    return CtxtTensor(s, bsgs_diagonals(e, op.get(), s, true, true));
}

// multMatMat<Ciphertext> -- MatrixUtils.cpp:1307-1446, in two halves so that callers holding operands of different
// levels (a transposed tile sits one level lower) can run the transforms per group and the product loop on all of
// them together.  First half: sigma(A), tau(B), both brought to target + 2 (:1346-1361).
void ccmmPrepare(Env &e, const CtxtTensor &op1, const CtxtTensor &op2, int target_level, Ciphertext &sa_out, Ciphertext &tb_out) {
    require_product_shapes(op1, op2);
    const i64 num_rows = op1.getHeight(), num_cols = op2.getWidth(), width = op1.getBlockWidth();
    const i64 num_k = ceil_pow2(op1.getWidth());
    if (std::min(op1.getLevel(), op2.getLevel()) < target_level + 3) throw std::invalid_argument("[multMatMat] level too low");
    const TileTensorShape sa(num_rows, num_k, width), sb(num_k, num_cols, width);
    const int lvl = target_level + 2;
    if (e.mode == kLazy) { // transforms at the lowest level that still leaves target + 2: far fewer limbs to transform
        sa_out = diagonalToColumn(e, CtxtTensor(sa, e.ev.levelDown(op1.get(), target_level + 3))).get();
        tb_out = diagonalToRow(e, CtxtTensor(sb, e.ev.levelDown(op2.get(), target_level + 3))).get();
        return;
    }
    sa_out = e.ev.levelDown(diagonalToColumn(e, CtxtTensor(sa, op1.get())).get(), lvl);
    tb_out = e.ev.levelDown(diagonalToRow(e, CtxtTensor(sb, op2.get())).get(), lvl);
}
// Second half: the k = 0 term, the shift-mask-tensor loop, relinearise, rescale, add (:1376-1443).
CtxtTensor ccmmCore(Env &e, Ciphertext a, Ciphertext b, i64 num_rows, i64 inner, i64 num_cols, i64 width, int target_level) {
    const i64 num_k = ceil_pow2(inner);
    const TileTensorShape sa(num_rows, num_k, width), sb(num_k, num_cols, width);
    const int lvl = target_level + 2;
    if (a.getLevel() != lvl || b.getLevel() != lvl) throw std::invalid_argument("[multMatMat] operands of the product loop must sit at target + 2");
    const i64 rows_tmp = num_k > num_rows ? num_k : ceil_pow2(num_rows), cols_tmp = num_k > num_cols ? num_k : ceil_pow2(num_cols);
    Ciphertext res = e.ev.mult(a, b);
    Ciphertext acc;
    if (e.mode == kLazy) {
        const Hoisted ha = e.ev.decompose(a), hb = e.ev.decompose(b);
        const i64 group = loop_group(a);
        for (i64 i0 = 1; i0 < num_k; i0 += group) {
            std::vector<WrappedCopy> wa, wb;
            for (i64 i = i0; i < std::min(num_k, i0 + group); ++i) {
                wa.push_back(wrapped_copy(e, false, sa, i, lvl, i, i - cols_tmp));
                wb.push_back(wrapped_copy(e, true, sb, i, lvl, i * width, (i - rows_tmp) * width));
            }
            Ciphertext ak = assemble_lazy(e, a, ha, wa), bk = assemble_lazy(e, b, hb, wb);
            e.ev.tensorAccumulateGroups(acc, ak, bk, (int)wa.size());
        }
    } else if (e.mode >= kDirect) {
        const Hoisted ha = e.ev.decompose(a), hb = e.ev.decompose(b);
        for (i64 i = 1; i < num_k; ++i) {
            Ciphertext ai = e.ev.leftRotate(a, ha, i), aw = e.ev.leftRotate(a, ha, i - cols_tmp);
            Ciphertext bi = e.ev.leftRotate(b, hb, i * width), bw = e.ev.leftRotate(b, hb, (i - rows_tmp) * width);
            Ciphertext ak = e.ev.assemble(ai, col_wrap(e, sa, 2 * i + 1, lvl), aw, col_wrap(e, sa, 2 * i, lvl));
            Ciphertext bk = e.ev.assemble(bi, row_wrap(e, sb, 2 * i + 1, lvl), bw, row_wrap(e, sb, 2 * i, lvl));
            e.ev.tensorAccumulate(acc, ak, bk);
        }
    } else {
        a = e.ev.leftRotate(a, 1);
        b = e.ev.leftRotate(b, width);
        Ciphertext a_wrap = e.ev.rightRotate(a, cols_tmp), b_wrap = e.ev.rightRotate(b, rows_tmp * width);
        for (i64 i = 1; i < num_k; ++i) {
            if (i > 1) {
                a = e.ev.leftRotate(a, 1); a_wrap = e.ev.leftRotate(a_wrap, 1);
                b = e.ev.leftRotate(b, width); b_wrap = e.ev.leftRotate(b_wrap, width);
            }
            Ciphertext ak = e.ev.assemble(a, col_wrap(e, sa, 2 * i + 1, lvl), a_wrap, col_wrap(e, sa, 2 * i, lvl));
            Ciphertext bk = e.ev.assemble(b, row_wrap(e, sb, 2 * i + 1, lvl), b_wrap, row_wrap(e, sb, 2 * i, lvl));
            e.ev.tensorAccumulate(acc, ak, bk);
        }
    }
    res = e.ev.add(res, e.ev.rescale(e.ev.relinearize(acc)));
    return CtxtTensor(TileTensorShape(num_rows, num_cols, width), std::move(res));
}
CtxtTensor multMatMatCC(Env &e, const CtxtTensor &op1, const CtxtTensor &op2, int target_level) {
    Ciphertext a, b;
    ccmmPrepare(e, op1, op2, target_level, a, b);
    return ccmmCore(e, std::move(a), std::move(b), op1.getHeight(), op1.getWidth(), op2.getWidth(), op1.getBlockWidth(), target_level);
}

// multMatMat<Plaintext> (HEMMer::singleMatMul) -- MatrixUtils.cpp:1448-1570: ciphertext x plaintext without reuse.  The right
// operand is decoded, tau-transformed in the clear (diagonalToRow<Plaintext>, :1072-1098), encoded at target + 2 and then
// shifted by slot rotations of the plaintext; its row wrap uses plaintext x mask products as the reference does.
CtxtTensor multMatMatCP(Env &e, const CtxtTensor &op1, const PtxtTensor &op2, int target_level) {
    if (op1.getWidth() != op2.getHeight()) throw std::invalid_argument("[getCommonInsideLength] different inside length.");
    if (op1.getBlockWidth() != op2.getBlockWidth()) throw std::invalid_argument("[getCommonBlockWidth] different block width");
    const i64 num_rows = op1.getHeight(), num_cols = op2.getWidth(), width = op1.getBlockWidth();
    const i64 num_k = ceil_pow2(op1.getWidth());
    if (op1.getLevel() < target_level + 3) throw std::invalid_argument("[multMatMat] level too low");
    const TileTensorShape sa(num_rows, num_k, width), sb(num_k, num_cols, width);
    const int lvl = target_level + 2;
    Ciphertext a = e.ev.levelDown(diagonalToColumn(e, CtxtTensor(sa, op1.get())).get(), lvl);
    const Message msg = e.ev.decode(op2.get(), (size_t)e.slots);
    Message tau((size_t)e.slots);
    for (i64 i = 0; i < sb.getNumRows(); ++i)
        for (i64 j = 0; j < sb.getNumCols(); ++j) {
            const size_t dst = (size_t)(((i - j + sb.getNumRows()) % sb.getNumRows()) * width + j), src = (size_t)(i * width + j);
            tau.re[dst] = msg.re[src]; tau.im[dst] = msg.im[src];
            if (width != sb.getNumCols()) { tau.re[dst + sb.getNumCols()] = msg.re[src + sb.getNumCols()]; tau.im[dst + sb.getNumCols()] = msg.im[src + sb.getNumCols()]; }
        }
    Plaintext b = e.ev.encode(tau, lvl);
    const i64 rows_tmp = num_k > num_rows ? num_k : ceil_pow2(num_rows), cols_tmp = num_k > num_cols ? num_k : ceil_pow2(num_cols);
    Ciphertext res = e.ev.mult(a, b);
    a = e.ev.leftRotate(a, 1);
    b = e.ev.leftRotate(b, width);
    Ciphertext a_wrap = e.ev.rightRotate(a, cols_tmp);
    Plaintext b_wrap = e.ev.leftRotate(b, -rows_tmp * width);
    Ciphertext acc;
    for (i64 i = 1; i < num_k; ++i) {
        if (i > 1) {
            a = e.ev.leftRotate(a, 1); a_wrap = e.ev.leftRotate(a_wrap, 1);
            b = e.ev.leftRotate(b, width); b_wrap = e.ev.leftRotate(b_wrap, width);
        }
        Ciphertext ak = e.ev.assemble(a, col_wrap(e, sa, 2 * i + 1, lvl), a_wrap, col_wrap(e, sa, 2 * i, lvl));
        Plaintext bk = e.ev.add(e.ev.mult(b, row_wrap(e, sb, 2 * i + 1, lvl)), e.ev.mult(b_wrap, row_wrap(e, sb, 2 * i, lvl)));
        Ciphertext term = e.ev.mult(ak, bk);
        acc = acc.empty() ? std::move(term) : e.ev.add(acc, term);
    }
    return CtxtTensor(TileTensorShape(num_rows, num_cols, width), e.ev.add(res, acc));
}

// multPackedMatMat -- MatrixUtils.cpp:1100-1216
CtxtTensor multPackedMatMat(Env &e, const CtxtTensor &op1, const CtxtTensor &op2, int target_level) {
    require_product_shapes(op1, op2);
    const i64 num_rows = op1.getHeight(), num_cols = op2.getWidth(), width = op1.getBlockWidth();
    const i64 num_k = ceil_pow2(op1.getWidth());
    if (op1.getLevel() < target_level + 3 || op2.getLevel() < target_level + 2) throw std::invalid_argument("[multMatMat] level too low");
    const TileTensorShape sa(num_rows, num_k, width), sb(num_k, num_cols, width);
    const int lvl = target_level + 2;
    Ciphertext a = packedDiagonalToColumn(e, CtxtTensor(sa, e.ev.levelDown(op1.get(), target_level + 3))).get();
    Ciphertext b = packedDiagonalToRow(e, CtxtTensor(sb, e.ev.levelDown(op2.get(), target_level + 2))).get();
    const i64 cols_tmp = num_k > num_cols ? num_k : ceil_pow2(num_cols);
    Ciphertext res = e.ev.mult(a, b);
    Ciphertext acc;
    if (e.mode >= kDirect) {
        const Hoisted ha = e.ev.decompose(a), hb = e.ev.decompose(b);
        for (i64 i = 1; i < num_k / 2; ++i) {
            Ciphertext ai = e.ev.leftRotate(a, ha, 2 * i), aw = e.ev.leftRotate(a, ha, 2 * i - cols_tmp);
            Ciphertext bi = e.ev.leftRotate(b, hb, 2 * i * width);
            Ciphertext ak = e.ev.assemble(ai, col_wrap(e, sa, 4 * i + 1, lvl), aw, col_wrap(e, sa, 4 * i, lvl));
            e.ev.tensorAccumulate(acc, ak, bi);
        }
    } else {
        a = e.ev.leftRotate(a, 2);
        b = e.ev.leftRotate(b, 2 * width);
        Ciphertext a_wrap = e.ev.rightRotate(a, cols_tmp);
        for (i64 i = 1; i < num_k / 2; ++i) {
            if (i > 1) {
                a = e.ev.leftRotate(a, 2); a_wrap = e.ev.leftRotate(a_wrap, 2);
                b = e.ev.leftRotate(b, 2 * width);
            }
            Ciphertext ak = e.ev.assemble(a, col_wrap(e, sa, 4 * i + 1, lvl), a_wrap, col_wrap(e, sa, 4 * i, lvl));
            e.ev.tensorAccumulate(acc, ak, b);
        }
    }
    res = e.ev.add(res, e.ev.rescale(e.ev.relinearize(acc)));
    return CtxtTensor(TileTensorShape(num_rows, num_cols, width), std::move(res));
}
// multPackedMatMatPre -- MatrixUtils.cpp:1218-1226
CtxtTensor multPackedMatMatPre(Env &e, const CtxtTensor &a, int target_level) {
    return packedDiagonalToColumn(e, CtxtTensor(a.getShape(), e.ev.levelDown(a.get(), target_level + 3)));
}
// multPackedMatMatPreRot -- MatrixUtils.cpp:1228-1264; the shifted copies come back as one batch
Ciphertext multPackedMatMatPreRot(Env &e, const CtxtTensor &in, int target_level) {
    const i64 num_rows = in.getHeight();
    const int lvl = target_level + 2;
    std::vector<Ciphertext> copies;
    copies.push_back(e.ev.levelDownOne(in.get()));
    if (e.mode >= kDirect) {
        const Hoisted h = e.ev.decompose(in.get());
        for (i64 i = 1; i < num_rows / 2; ++i) {
            Ciphertext ai = e.ev.leftRotate(in.get(), h, 2 * i), aw = e.ev.leftRotate(in.get(), h, 2 * i - num_rows);
            copies.push_back(e.ev.assemble(ai, col_wrap(e, in.getShape(), 4 * i + 1, lvl), aw, col_wrap(e, in.getShape(), 4 * i, lvl)));
        }
        return e.ev.stack(copies);
    }
    Ciphertext a = e.ev.leftRotate(in.get(), 2);
    Ciphertext a_wrap = e.ev.rightRotate(a, num_rows);
    for (i64 i = 1; i < num_rows / 2; ++i) {
        if (i > 1) { a = e.ev.leftRotate(a, 2); a_wrap = e.ev.leftRotate(a_wrap, 2); }
        copies.push_back(e.ev.assemble(a, col_wrap(e, in.getShape(), 4 * i + 1, lvl), a_wrap, col_wrap(e, in.getShape(), 4 * i, lvl)));
    }
    return e.ev.stack(copies);
}
// multPackedMatMatPreRev -- MatrixUtils.cpp:1266-1274
CtxtTensor multPackedMatMatPreRev(Env &e, const CtxtTensor &b, int target_level) {
    return packedDiagonalToRow(e, CtxtTensor(b.getShape(), e.ev.levelDown(b.get(), target_level + 2)));
}
// multPackedMatMatCCReuse -- MatrixUtils.cpp:1276-1305 (relinearised and rescaled)
CtxtTensor multPackedMatMatCCReuse(Env &e, const Ciphertext &pre, const CtxtTensor &tb) {
    const i64 width = tb.getBlockWidth();
    Ciphertext b = tb.get(), acc;
    const int count = pre.getBatch();
    const Hoisted h = e.mode >= kDirect ? e.ev.decompose(tb.get()) : Hoisted();
    for (int i = 0; i < count; ++i) {
        if (i > 0) b = e.mode >= kDirect ? e.ev.leftRotate(tb.get(), h, (i64)i * 2 * width) : e.ev.leftRotate(b, 2 * width);
        e.ev.tensorAccumulate(acc, e.ev.slice(pre, i), b);
    }
    return CtxtTensor(tb.getShape(), e.ev.rescale(e.ev.relinearize(acc)));
}

// multMatMatPre -- MatrixUtils.cpp:1572-1610; the `rows` shifted copies come back as one batch
Ciphertext multMatMatPre(Env &e, const CtxtTensor &in, int target_level) {
    const i64 num_rows = in.getHeight();
    const int lvl = target_level + 2;
    CtxtTensor s = diagonalToColumn(e, CtxtTensor(in.getShape(), e.ev.levelDown(in.get(), target_level + 3)));
    std::vector<Ciphertext> copies;
    copies.push_back(e.ev.levelDownOne(s.get()));
    if (e.mode == kLazy) {
        const Hoisted h = e.ev.decompose(s.get());
        const i64 group = loop_group(s.get());
        for (i64 i0 = 1; i0 < num_rows; i0 += group) { // a group of copies is already laid out copy-major, as stack() lays them
            std::vector<WrappedCopy> w;
            for (i64 i = i0; i < std::min(num_rows, i0 + group); ++i) w.push_back(wrapped_copy(e, false, s.getShape(), i, lvl, i, i - num_rows));
            copies.push_back(assemble_lazy(e, s.get(), h, w));
        }
        return e.ev.concat(copies);
    }
    if (e.mode >= kDirect) {
        const Hoisted h = e.ev.decompose(s.get());
        for (i64 i = 1; i < num_rows; ++i) {
            Ciphertext ai = e.ev.leftRotate(s.get(), h, i), aw = e.ev.leftRotate(s.get(), h, i - num_rows);
            copies.push_back(e.ev.assemble(ai, col_wrap(e, s.getShape(), 2 * i + 1, lvl), aw, col_wrap(e, s.getShape(), 2 * i, lvl)));
        }
        return e.ev.stack(copies);
    }
    Ciphertext a = e.ev.leftRotate(s.get(), 1);
    Ciphertext a_wrap = e.ev.rightRotate(a, num_rows);
    for (i64 i = 1; i < num_rows; ++i) {
        if (i > 1) { a = e.ev.leftRotate(a, 1); a_wrap = e.ev.leftRotate(a_wrap, 1); }
        copies.push_back(e.ev.assemble(a, col_wrap(e, s.getShape(), 2 * i + 1, lvl), a_wrap, col_wrap(e, s.getShape(), 2 * i, lvl)));
    }
    return e.ev.stack(copies);
}
// multMatMatReUse -- MatrixUtils.cpp:1612-1639: one fused pass over the shifted copies
CtxtTensor multMatMatReUse(Env &e, const Ciphertext &pre, const PtxtTensor &w) {
    if (w.getLevel() != pre.getLevel()) throw std::invalid_argument("[multMatMatReUse] plaintext level differs from the ciphertexts'");
    return CtxtTensor(w.getShape(), e.ev.matmul(pre, w.get(), w.getBlockWidth()));
}
// multMatMatPreRev -- MatrixUtils.cpp:1641-1649
CtxtTensor multMatMatPreRev(Env &e, const CtxtTensor &b, int target_level) {
    return diagonalToRow(e, CtxtTensor(b.getShape(), e.ev.levelDown(b.get(), target_level + 2)));
}
// multMatMatCCReUse -- MatrixUtils.cpp:1651-1679 (relinearised, not rescaled)
CtxtTensor multMatMatCCReUse(Env &e, const Ciphertext &pre, const CtxtTensor &tb) {
    const i64 width = tb.getBlockWidth();
    Ciphertext b = tb.get(), acc;
    const int count = pre.getBatch();
    const Hoisted h = e.mode >= kDirect ? e.ev.decompose(tb.get()) : Hoisted();
    for (int i = 0; i < count; ++i) {
        if (i > 0) b = e.mode >= kDirect ? e.ev.leftRotate(tb.get(), h, (i64)i * width) : e.ev.leftRotate(b, width);
        e.ev.tensorAccumulate(acc, e.ev.slice(pre, i), b);
    }
    return CtxtTensor(tb.getShape(), e.ev.relinearize(acc));
}

// ---- LoRA low-rank products -- MatrixUtils.cpp:1681-1996 --------------------------------------------------
// One factor has only low_dim columns (or rows).  Its transform then has low_dim diagonals and the product loop
// low_dim terms; the other terms of the inner sum are folded by doubling trees of rotate-and-add, here on the
// thin operand (so that every low_dim-wide block of it carries the term it meets in the loop) and, afterwards,
// in HEMMer::repackTo*.  The operation order is that of the reference functions.
namespace {
void require_low_rank(const CtxtTensor &a, const CtxtTensor &b, int target_level, i64 low_dim) {
    if (low_dim < 1 || (low_dim & (low_dim - 1))) throw std::invalid_argument("[lowRank] low_dim must be a power of two");
    if (std::min(a.getLevel(), b.getLevel()) < target_level + 3) throw std::invalid_argument("[lowRank] level too low");
}
// x + rot(x, +-step * i) for i = low_dim, 2 low_dim, ... < end; bit j of `pos` picks the direction of round j
Ciphertext fold_tree(Env &e, Ciphertext x, i64 low_dim, i64 end, i64 step, i64 pos, bool even_goes_right) {
    for (i64 i = low_dim; i < end; i <<= 1, pos /= 2) {
        const bool right = (pos % 2 == 0) == even_goes_right;
        x = e.ev.add(x, right ? e.ev.rightRotate(x, i * step) : e.ev.leftRotate(x, i * step));
    }
    return x;
}
// k = 0 term plus the low_dim - 1 shifted terms (the common tail of the three reference functions)
CtxtTensor low_rank_tail(Env &e, Ciphertext a, Ciphertext b, const TileTensorShape &s1, const TileTensorShape &s2, i64 width, i64 low_dim, int target_level) {
    const int lvl = target_level + 2;
    const i64 num_rows = s1.getNumRows();
    Ciphertext res = e.ev.mult(a, b);
    if (low_dim > 1) {
        a = e.ev.leftRotate(a, 1);
        b = e.ev.leftRotate(b, width);
        Ciphertext a_wrap = e.ev.rightRotate(a, width / 2), b_wrap = e.ev.rightRotate(b, num_rows * width);
        Ciphertext acc;
        for (i64 i = 1; i < low_dim; ++i) {
            if (i > 1) {
                a = e.ev.leftRotate(a, 1); a_wrap = e.ev.leftRotate(a_wrap, 1);
                b = e.ev.leftRotate(b, width); b_wrap = e.ev.leftRotate(b_wrap, width);
            }
            Ciphertext ak = e.ev.assemble(a, col_wrap(e, s1, 2 * i + 1, lvl), a_wrap, col_wrap(e, s1, 2 * i, lvl));
            Ciphertext bk = e.ev.assemble(b, row_wrap(e, s2, 2 * i + 1, lvl), b_wrap, row_wrap(e, s2, 2 * i, lvl));
            e.ev.tensorAccumulate(acc, ak, bk);
        }
        res = e.ev.add(res, e.ev.rescale(e.ev.relinearize(acc)));
    }
    return CtxtTensor(TileTensorShape(s1.getNumRows(), s2.getNumCols(), s2.getBlockWidth()), std::move(res));
}
} // namespace

// multMatMatHighLow -- MatrixUtils.cpp:1681-1771
CtxtTensor multMatMatHighLow(Env &e, const CtxtTensor &op1, const CtxtTensor &op2, i64 in_col_block, int target_level, i64 low_dim) {
    require_low_rank(op1, op2, target_level, low_dim);
    const i64 width = op2.getBlockWidth();
    Ciphertext a = diagonalToColumn(e, CtxtTensor(op1.getShape(), e.ev.levelDown(op1.get(), target_level + 3))).get();
    Ciphertext b = diagonalToRow(e, CtxtTensor(TileTensorShape(op2.getHeight(), low_dim, width), e.ev.levelDown(op2.get(), target_level + 3))).get();
    i64 col_pos = in_col_block;
    for (i64 i = low_dim; i < width / 2; i <<= 1, col_pos /= 2) {
        if (col_pos % 2 == 0) {
            b = e.ev.add(b, e.ev.rightRotate(e.ev.leftRotate(b, i * width), i));
        } else {
            Ciphertext side = e.ev.leftRotate(b, i);
            b = e.ev.add(e.ev.leftRotate(b, i * width), side);
        }
    }
    return low_rank_tail(e, std::move(a), std::move(b), op1.getShape(), op2.getShape(), width, low_dim, target_level);
}
// multMatMatLowHigh -- MatrixUtils.cpp:1773-1879
CtxtTensor multMatMatLowHigh(Env &e, const CtxtTensor &op1, const CtxtTensor &op2, i64 in_row_block, int target_level, i64 low_dim) {
    require_low_rank(op1, op2, target_level, low_dim);
    if (op1.getBlockWidth() != op2.getBlockWidth()) throw std::invalid_argument("[getCommonBlockWidth] different block width");
    const i64 width = op1.getBlockWidth();
    Ciphertext a = fold_tree(e, e.ev.levelDown(op1.get(), target_level + 3), low_dim, width / 2, width, in_row_block, true);
    a = diagonalToColumn(e, CtxtTensor(op1.getShape(), std::move(a))).get();
    Ciphertext b = diagonalToRow(e, CtxtTensor(op2.getShape(), e.ev.levelDown(op2.get(), target_level + 3))).get();
    return low_rank_tail(e, std::move(a), std::move(b), op1.getShape(), op2.getShape(), width, low_dim, target_level);
}
// multMatMatLowLow -- MatrixUtils.cpp:1881-1996
CtxtTensor multMatMatLowLow(Env &e, const CtxtTensor &op1, const CtxtTensor &op2, i64 in_col_block, i64 in_row_block, int target_level, i64 low_dim) {
    require_low_rank(op1, op2, target_level, low_dim);
    if (op1.getBlockWidth() != op2.getBlockWidth()) throw std::invalid_argument("[getCommonBlockWidth] different block width");
    const i64 width = op1.getBlockWidth();
    Ciphertext a = diagonalToColumn(e, CtxtTensor(TileTensorShape(op1.getHeight(), low_dim, width), e.ev.levelDown(op1.get(), target_level + 3))).get();
    Ciphertext b = diagonalToRow(e, CtxtTensor(TileTensorShape(low_dim, op2.getWidth(), width), e.ev.levelDown(op2.get(), target_level + 3))).get();
    // the reference interleaves the two trees round by round; they touch different ciphertexts, so running one
    // after the other leaves every bit as it was
    a = fold_tree(e, std::move(a), low_dim, width / 2, 1, in_col_block, true);
    b = fold_tree(e, std::move(b), low_dim, width / 2, width, in_row_block, true);
    return low_rank_tail(e, std::move(a), std::move(b), op1.getShape(), op2.getShape(), width, low_dim, target_level);
}

} // namespace sched
} // namespace HELLM
