// CPU ORACLE -- TEST INFRASTRUCTURE ONLY (see ckks_oracle.hpp for scope and "parity unpinned").
//
// Restatement of the reference's matrix-multiplication schedules over the oracle's
// primitives.  Each function names the reference function it follows
// (ciphertext/src/MatrixUtils.cpp and ciphertext/src/HEMMer.cpp); operation order is
// kept exactly, because the ciphertext residues depend on it.  The slot count is a
// parameter here (the reference hard-codes 2^15, MatrixUtils.cpp:84) and the tile side
// of the HEMMer-level masks is d = sqrt(slots/2) (the reference hard-codes 128,
// ModelArgs.hpp:33-72).
#pragma once
#include "ckks_oracle.hpp"

namespace orc {

using Message = std::vector<cplx>;

// TileTensorShape -- include/HELLM/HETensor.hpp:16-44
struct Shape {
    i64 rows = 0, cols = 0, width = 0;
    Shape() {}
    Shape(i64 r, i64 c, i64 w) : rows(r), cols(c), width(w) {}
    Shape(i64 r, i64 c) : rows(r), cols(c) { i64 i = 1; while (c > i) i <<= 1; width = i; }
    bool operator<(const Shape &o) const { return std::tie(rows, cols, width) < std::tie(o.rows, o.cols, o.width); }
};
// HETensor<Ciphertext> / HETensor<Plaintext> -- include/HELLM/HETensor.hpp:46-86
struct CtT { Ct ct; Shape sh; };
struct PtT { Pt pt; Shape sh; };

inline Message msg_rotate_right(const Message &m, i64 r) {
    const i64 n = (i64)m.size(); r %= n; if (r < 0) r += n;
    Message o(m.size());
    for (i64 i = 0; i < n; ++i) o[(size_t)((i + r) % n)] = m[(size_t)i];
    return o;
}
inline Message msg_rotate_left(const Message &m, i64 r) { return msg_rotate_right(m, -r); }

// A cleartext mask with its per-level encodings (the reference re-encodes a Message inside every
// eval.mult(ct, Message); encoding is deterministic, so caching changes no bit).
struct Mask {
    Message msg;
    std::map<int, Pt> enc;
};

struct Hemmer {
    Context &cx; Evaluator &ev;
    const i64 slots;
    i64 tile; // side of the square tile that fills half the slots of a two-tile ciphertext

    std::map<Shape, std::map<i64, Mask>> diagonal_mask_, horizontal_mask_, vertical_mask_, packed_horizontal_mask_, packed_vertical_mask_;
    std::map<std::pair<int, Shape>, std::vector<Pt>> row_mask_, col_mask_;
    Mask col_mask_even_, row_mask_even_, mask_left_half_;
    std::map<int, Pt> mask_matmul_;

    // 0: the reference's rotation sequence (each shifted copy is the previous one rotated once more).
    // 1: "direct" variant -- every shifted copy is one rotation of the transformed operand itself, rot(x, k).
    //    Same slots, different ciphertext bits (fewer chained key switches).  The CUDA library implements the
    //    same variant with hoisting; both variants are compared bit for bit.
    // 2: as 1, and the masked pair of rotations that makes a wrapped copy is one Evaluator::assemble_rot (one
    //    division by P * q_level for the pair) in the product loop and in multMatMatPre; multMatMat brings its operands
    //    down to target + 3 BEFORE sigma / tau instead of after (MatrixUtils.cpp:1346-1361 transforms at the operands'
    //    level), the order multMatMatPre (:1583) and the low-rank products (:1692) use; the masked sums of the
    //    baby-step / giant-step transforms are rescaled once per sum instead of once per term (MaskedSum), and their
    //    giant-step rotations share one ModDown (GiantSum).
    int mode = 0;

    Hemmer(Context &c, Evaluator &e) : cx(c), ev(e), slots(c.slots) {
        tile = 1; while (2 * tile * tile < slots) tile <<= 1;
        gen_axis_masks();
    }

    // ---------------- primitive wrappers ----------------
    Ct rotL(const Ct &x, i64 r) { ev.gen_rot_key(r); return ev.rotate(x, r); }
    Ct rotR(const Ct &x, i64 r) { return rotL(x, -r); }
    const Pt &enc_mask(Mask &m, int level) {
        auto it = m.enc.find(level);
        if (it == m.enc.end()) it = m.enc.emplace(level, ev.encode(m.msg.data(), m.msg.size(), level)).first;
        return it->second;
    }
    // eval.mult(ct, Message) -- HomEvaluator.hpp:287-289
    Ct mult_msg(const Ct &x, Mask &m) { return ev.mul_pt(x, enc_mask(m, x.level)); }
    // One masked sum of a baby-step / giant-step transform.  The reference rescales every product and adds the
    // results (eval.mult(ct, Message) per term); schedule 2 adds the un-rescaled products and rescales the sum once.
    struct MaskedSum {
        Hemmer &h; Ct acc; bool any = false;
        explicit MaskedSum(Hemmer &hh) : h(hh) {}
        void add(const Ct &x, Mask &m) {
            Ct t = h.mode == 2 ? h.ev.mul_pt_norescale(x, h.enc_mask(m, x.level)) : h.mult_msg(x, m);
            acc = any ? h.ev.add(acc, t) : t;
            any = true;
        }
        Ct result() { return h.mode == 2 ? h.ev.rescale(acc) : acc; }
    };

    // The giant-step rotations of a transform and their sum.  Schedule 2 adds the key-switch inner products of all
    // giant steps in the extended basis and applies ONE ModDown (Evaluator::rotate_sum); the other schedules rotate
    // every part on its own and add, in the order the reference does.
    struct GiantSum {
        Hemmer &h; std::vector<Ct> parts; std::vector<i64> steps; Ct res; bool any = false;
        explicit GiantSum(Hemmer &hh) : h(hh) {}
        void add(Ct part, i64 left_steps) {
            if (h.mode == 2) { parts.push_back(std::move(part)); steps.push_back(left_steps); return; }
            Ct t = (left_steps % h.slots) ? h.rotL(part, left_steps) : part;
            res = any ? h.ev.add(res, t) : t;
            any = true;
        }
        Ct result() {
            if (h.mode != 2) return res;
            std::vector<const Ct *> ptr;
            for (size_t i = 0; i < parts.size(); ++i) { h.ev.gen_rot_key(steps[i]); ptr.push_back(&parts[i]); }
            return h.ev.rotate_sum(ptr, steps);
        }
    };

    // ---------------- TransformMask generators ----------------
    // generateDiagoanlMask -- MatrixUtils.cpp:90-127
    std::map<i64, Mask> &get_diagonal_mask(const Shape &s) {
        auto &mp = diagonal_mask_[s];
        if (!mp.empty()) return mp;
        const i64 num_rows = s.rows, num_cols = s.cols, width = s.width;
        const i64 num_mask = num_rows + num_cols - 1;
        const i64 bs = (i64)std::ceil(std::sqrt((double)num_mask));
        const i64 gs = (i64)std::ceil((double)num_mask / (double)bs);
        for (i64 i = 0; i < gs; i++) {
            const i64 rot_num = i * bs * (width - 1);
            for (i64 j = 0; j < bs; j++) {
                const i64 idx = 1 - num_rows + i * bs + j;
                if (idx >= num_cols) break;
                Message msg((size_t)slots, cplx(0, 0));
                const i64 start_row = (idx < 0) ? -idx : 0, start_col = (idx < 0) ? 0 : idx;
                for (i64 row = start_row, col = start_col; row < num_rows && col < num_cols; row++, col++) {
                    msg[(size_t)(row * width + col)] = 1;
                    if (width != num_cols) msg[(size_t)(row * width + num_rows + col)] = 1;
                }
                mp[idx].msg = msg_rotate_right(msg, rot_num);
            }
        }
        return mp;
    }
    void fill_blocks(Message &msg, i64 row, i64 col, const Shape &s, double v = 1.0) {
        const i64 height = slots / s.width;
        for (i64 rb = 0; rb < height; rb += s.rows)
            for (i64 cb = 0; cb < s.width; cb += s.cols) msg[(size_t)((rb + row) * s.width + cb + col)] = v;
    }
    // generateHorizontalMask -- MatrixUtils.cpp:129-217
    std::map<i64, Mask> &get_horizontal_mask(const Shape &s) {
        auto &mp = horizontal_mask_[s];
        if (!mp.empty()) return mp;
        const i64 num_rows = s.rows, num_cols = s.cols;
        const i64 sub_dim = (num_rows > num_cols) ? num_cols : num_rows;
        const i64 bs = (i64)std::ceil(std::sqrt((double)(2 * sub_dim - 1)));
        const i64 gs = (i64)std::ceil((double)(sub_dim - 1) / (double)bs);
        for (i64 i = 0; i < gs; i++) {
            if (i == 0) {
                Message msg((size_t)slots, cplx(0, 0));
                for (i64 row = 0; row < num_rows; row += sub_dim)
                    for (i64 col = 0; col < num_cols; col++) fill_blocks(msg, row, col, s);
                mp[0].msg = msg;
            }
            const i64 rot_num = i * bs;
            for (i64 j = 0; j < bs; j++) {
                const i64 idx = 1 + i * bs + j - num_cols;
                if (idx >= sub_dim - num_cols) break;
                Message msg((size_t)slots, cplx(0, 0));
                for (i64 row = num_cols + idx; row < num_rows; row += sub_dim)
                    for (i64 col = -idx; col < num_cols; col++) fill_blocks(msg, row, col, s);
                mp[idx].msg = msg_rotate_right(msg, rot_num - num_cols);
            }
            for (i64 j = 0; j < bs; j++) {
                const i64 idx = 1 + i * bs + j;
                if (idx >= sub_dim) break;
                Message msg((size_t)slots, cplx(0, 0));
                for (i64 row = idx; row < num_rows; row += sub_dim)
                    for (i64 col = 0; col < num_cols - idx; col++) fill_blocks(msg, row, col, s);
                mp[idx].msg = msg_rotate_right(msg, rot_num);
            }
        }
        return mp;
    }
    // generateVerticalMask -- MatrixUtils.cpp:330-419
    std::map<i64, Mask> &get_vertical_mask(const Shape &s) {
        auto &mp = vertical_mask_[s];
        if (!mp.empty()) return mp;
        const i64 num_rows = s.rows, num_cols = s.cols, width = s.width;
        const i64 sub_dim = (num_cols > num_rows) ? num_rows : num_cols;
        const i64 bs = (i64)std::ceil(std::sqrt((double)(2 * sub_dim - 1)));
        const i64 gs = (i64)std::ceil((double)(sub_dim - 1) / (double)bs);
        for (i64 i = 0; i < gs; i++) {
            if (i == 0) {
                Message msg((size_t)slots, cplx(0, 0));
                for (i64 col = 0; col < num_cols; col += sub_dim)
                    for (i64 row = 0; row < num_rows; row++) fill_blocks(msg, row, col, s);
                mp[0].msg = msg;
            }
            const i64 rot_num = i * bs * width;
            for (i64 j = 0; j < bs; j++) {
                const i64 idx = 1 + i * bs + j - num_rows;
                if (idx >= sub_dim - num_rows) break;
                Message msg((size_t)slots, cplx(0, 0));
                for (i64 col = num_rows + idx; col < num_cols; col += sub_dim)
                    for (i64 row = -idx; row < num_rows; row++) fill_blocks(msg, row, col, s);
                mp[idx].msg = msg_rotate_left(msg, num_rows * width - rot_num);
            }
            for (i64 j = 0; j < bs; j++) {
                const i64 idx = 1 + i * bs + j;
                if (idx >= sub_dim) break;
                Message msg((size_t)slots, cplx(0, 0));
                for (i64 col = idx; col < num_cols; col += sub_dim)
                    for (i64 row = 0; row < num_rows - idx; row++) fill_blocks(msg, row, col, s);
                mp[idx].msg = msg_rotate_right(msg, rot_num);
            }
        }
        return mp;
    }
    void fill_packed(Message &msg, i64 row, i64 col, i64 width, i64 num_cols, double v) {
        for (i64 dr = 0; dr < 2; ++dr)
            for (i64 dc = 0; dc < 2; ++dc) {
                msg[(size_t)((2 * row + dr) * width + (2 * col + dc))] = v;
                if (width != num_cols) msg[(size_t)((2 * row + dr) * width + 2 * num_cols + (2 * col + dc))] = v;
            }
    }
    // generatePackedHorizontalMask -- MatrixUtils.cpp:219-328 (value 0.5)
    std::map<i64, Mask> &get_packed_horizontal_mask(const Shape &s) {
        auto &mp = packed_horizontal_mask_[s];
        if (!mp.empty()) return mp;
        const i64 num_rows = s.rows / 2, num_cols = s.cols / 2, width = s.width;
        const i64 sub_dim = (num_rows > num_cols) ? num_cols : num_rows;
        const i64 bs = (i64)std::ceil(std::sqrt((double)(2 * sub_dim - 1)));
        const i64 gs = (i64)std::ceil((double)(sub_dim - 1) / (double)bs);
        for (i64 i = 0; i < gs; i++) {
            if (i == 0) {
                Message msg((size_t)slots, cplx(0, 0));
                for (i64 row = 0; row < num_rows; row += sub_dim)
                    for (i64 col = 0; col < num_cols; col++) fill_packed(msg, row, col, width, num_cols, 0.5);
                mp[0].msg = msg;
            }
            const i64 rot_num = 2 * i * bs;
            for (i64 j = 0; j < bs; j++) {
                const i64 idx = 1 + i * bs + j - num_cols;
                if (idx >= sub_dim - num_cols) break;
                Message msg((size_t)slots, cplx(0, 0));
                for (i64 row = num_cols + idx; row < num_rows; row += sub_dim)
                    for (i64 col = -idx; col < num_cols; col++) fill_packed(msg, row, col, width, num_cols, 0.5);
                mp[idx].msg = msg_rotate_right(msg, rot_num - 2 * num_cols);
            }
            for (i64 j = 0; j < bs; j++) {
                const i64 idx = 1 + i * bs + j;
                if (idx >= sub_dim) break;
                Message msg((size_t)slots, cplx(0, 0));
                for (i64 row = idx; row < num_rows; row += sub_dim)
                    for (i64 col = 0; col < num_cols - idx; col++) fill_packed(msg, row, col, width, num_cols, 0.5);
                mp[idx].msg = msg_rotate_right(msg, rot_num);
            }
        }
        return mp;
    }
    // generatePackedVerticalMask -- MatrixUtils.cpp:421-527 (value 1)
    std::map<i64, Mask> &get_packed_vertical_mask(const Shape &s) {
        auto &mp = packed_vertical_mask_[s];
        if (!mp.empty()) return mp;
        const i64 num_rows = s.rows / 2, num_cols = s.cols / 2, width = s.width;
        const i64 sub_dim = (num_cols > num_rows) ? num_rows : num_cols;
        const i64 bs = (i64)std::ceil(std::sqrt((double)(2 * sub_dim - 1)));
        const i64 gs = (i64)std::ceil((double)(sub_dim - 1) / (double)bs);
        for (i64 i = 0; i < gs; i++) {
            if (i == 0) {
                Message msg((size_t)slots, cplx(0, 0));
                for (i64 col = 0; col < num_cols; col += sub_dim)
                    for (i64 row = 0; row < num_rows; row++) fill_packed(msg, row, col, width, num_cols, 1.0);
                mp[0].msg = msg;
            }
            const i64 rot_num = 2 * i * bs * width;
            for (i64 j = 0; j < bs; j++) {
                const i64 idx = 1 + i * bs + j - num_rows;
                if (idx >= sub_dim - num_rows) break;
                Message msg((size_t)slots, cplx(0, 0));
                for (i64 col = num_rows + idx; col < num_cols; col += sub_dim)
                    for (i64 row = -idx; row < num_rows; row++) fill_packed(msg, row, col, width, num_cols, 1.0);
                mp[idx].msg = msg_rotate_left(msg, 2 * num_rows * width - rot_num);
            }
            for (i64 j = 0; j < bs; j++) {
                const i64 idx = 1 + i * bs + j;
                if (idx >= sub_dim) break;
                Message msg((size_t)slots, cplx(0, 0));
                for (i64 col = idx; col < num_cols; col += sub_dim)
                    for (i64 row = 0; row < num_rows - idx; row++) fill_packed(msg, row, col, width, num_cols, 1.0);
                mp[idx].msg = msg_rotate_right(msg, rot_num);
            }
        }
        return mp;
    }
    // generateRowMask -- MatrixUtils.cpp:529-552 (plaintexts at target_level, two per shift).  The wrap masks carry
    // the extra limbs of encode_ext so that schedule 2 can use them; their first target_level + 1 limbs are those
    // of encode().
    std::vector<Pt> &get_row_mask(const Shape &s, int target_level) {
        auto &v = row_mask_[{target_level, s}];
        if (!v.empty()) return v;
        for (i64 i = 0; i < s.rows; i++) {
            Message msg((size_t)slots, cplx(1, 0)), rev((size_t)slots, cplx(0, 0));
            for (i64 j = 0; j < slots; j++)
                if ((j / s.width) % s.rows < s.rows - i) { msg[(size_t)j] = 0; rev[(size_t)j] = 1; }
            v.push_back(ev.encode_ext(msg.data(), msg.size(), target_level));
            v.push_back(ev.encode_ext(rev.data(), rev.size(), target_level));
        }
        return v;
    }
    // generateColMask -- MatrixUtils.cpp:554-578
    std::vector<Pt> &get_col_mask(const Shape &s, int target_level) {
        auto &v = col_mask_[{target_level, s}];
        if (!v.empty()) return v;
        for (i64 i = 0; i < s.cols; i++) {
            Message msg((size_t)slots, cplx(1, 0)), rev((size_t)slots, cplx(0, 0));
            for (i64 j = 0; j < slots; j++)
                if (j % s.cols < s.cols - i) { msg[(size_t)j] = 0; rev[(size_t)j] = 1; }
            v.push_back(ev.encode_ext(msg.data(), msg.size(), target_level));
            v.push_back(ev.encode_ext(rev.data(), rev.size(), target_level));
        }
        return v;
    }

    // ---------------- MatrixTransformer ----------------
    // transpose<Ciphertext> -- MatrixUtils.cpp:671-739
    CtT transpose(const CtT &op) {
        const i64 num_cols = op.sh.rows, num_rows = op.sh.cols, width = op.sh.width;
        if (num_cols > width) throw std::invalid_argument("[transpose] num_cols > width.");
        Shape ms(num_rows, num_cols, width);
        auto &dm = get_diagonal_mask(ms);
        const i64 bs = (i64)std::ceil(std::sqrt((double)(num_rows + num_cols - 1)));
        const i64 gs = (i64)std::ceil((double)(num_rows + num_cols - 1) / (double)bs);
        const i64 gap = width - 1;
        std::vector<Ct> bs_rot((size_t)bs);
        if (mode >= 1) {
            for (i64 j = 0; j < bs; j++) bs_rot[(size_t)j] = rotL(op.ct, (j - (num_rows - 1)) * gap);
        } else {
            bs_rot[0] = rotR(op.ct, (num_rows - 1) * gap);
            for (i64 j = 1; j < bs; j++) bs_rot[(size_t)j] = rotL(bs_rot[(size_t)j - 1], gap);
        }
        GiantSum giant(*this);
        for (i64 i = 0; i < gs; i++) {
            i64 idx = 1 - num_rows + i * bs;
            MaskedSum sum(*this);
            sum.add(bs_rot[0], dm[idx]);
            for (i64 j = 1; j < bs; j++) {
                if (++idx >= num_cols) break;
                sum.add(bs_rot[(size_t)j], dm[idx]);
            }
            giant.add(sum.result(), (i * bs) * gap);
        }
        return CtT{giant.result(), ms};
    }
    // Shared body of diagonalToColumn (MatrixUtils.cpp:776-848, gap 1, main = cols),
    // diagonalToRow (:924-996, gap = width, main = rows), packedDiagonalToColumn (:850-922, gap 2,
    // main = cols/2) and packedDiagonalToRow (:998-1070, gap 2*width, main = rows/2).
    Ct bsgs_diagonal(const Ct &op, std::map<i64, Mask> &mask, i64 sub_dim, i64 main_dim, i64 gap) {
        const i64 bs = (i64)std::ceil(std::sqrt((double)(2 * sub_dim - 1)));
        const i64 gs = (i64)std::ceil((double)(sub_dim - 1) / (double)bs);
        std::vector<Ct> bs_rot((size_t)bs);
        if (mode >= 1) {
            for (i64 j = 0; j < bs; j++) bs_rot[(size_t)j] = rotL(op, (j + 1) * gap);
        } else {
            bs_rot[0] = rotL(op, gap);
            for (i64 j = 1; j < bs; j++) bs_rot[(size_t)j] = rotL(bs_rot[(size_t)j - 1], gap);
        }
        GiantSum giant(*this);
        giant.add(mult_msg(op, mask[0]), 0);
        for (i64 i = 0; i < gs; i++) {
            const i64 rot_num = i * bs * gap;
            i64 idx = 1 + i * bs - main_dim;
            MaskedSum neg(*this);
            neg.add(bs_rot[0], mask[idx]);
            for (i64 j = 1; j < bs; j++) {
                if (++idx >= sub_dim - main_dim) break;
                neg.add(bs_rot[(size_t)j], mask[idx]);
            }
            giant.add(neg.result(), -(main_dim * gap - rot_num));
            idx = 1 + i * bs;
            MaskedSum pos(*this);
            pos.add(bs_rot[0], mask[idx]);
            for (i64 j = 1; j < bs; j++) {
                if (++idx >= sub_dim) break;
                pos.add(bs_rot[(size_t)j], mask[idx]);
            }
            giant.add(pos.result(), rot_num);
        }
        return giant.result();
    }
    CtT diagonal_to_column(const CtT &op) {
        Shape ms(op.sh.rows, op.sh.cols, op.sh.width);
        return CtT{bsgs_diagonal(op.ct, get_horizontal_mask(ms), std::min(ms.rows, ms.cols), ms.cols, 1), ms};
    }
    CtT diagonal_to_row(const CtT &op) {
        Shape ms(op.sh.rows, op.sh.cols, op.sh.width);
        return CtT{bsgs_diagonal(op.ct, get_vertical_mask(ms), std::min(ms.rows, ms.cols), ms.rows, ms.width), ms};
    }
    CtT packed_diagonal_to_column(const CtT &op) {
        const i64 nr = op.sh.rows / 2, nc = op.sh.cols / 2;
        Shape ms(2 * nr, 2 * nc, op.sh.width);
        return CtT{bsgs_diagonal(op.ct, get_packed_horizontal_mask(ms), std::min(nr, nc), nc, 2), ms};
    }
    CtT packed_diagonal_to_row(const CtT &op) {
        const i64 nr = op.sh.rows / 2, nc = op.sh.cols / 2;
        Shape ms(2 * nr, 2 * nc, op.sh.width);
        return CtT{bsgs_diagonal(op.ct, get_packed_vertical_mask(ms), std::min(nr, nc), nr, 2 * ms.width), ms};
    }

    static i64 pow2_ceil(i64 v) { i64 p = 1; while (p < v) p <<= 1; return p; }
    void check_level(const Ct &a, const Ct &b) {
        // the reference refuses operands below 1 + minimum bootstrap level (MatrixUtils.cpp:1320-1324);
        // without bootstrapping the requirement is that the schedule's level budget fits.
        (void)a; (void)b;
    }

    // "assemble": rescale(x (.) pa + y (.) pb) -- MatrixUtils.cpp:1424-1427
    Ct assemble(const Ct &x, const Pt &pa, const Ct &y, const Pt &pb) {
        return ev.rescale(ev.add(ev.mul_pt_norescale(x, pa), ev.mul_pt_norescale(y, pb)));
    }

    // multMatMat<Ciphertext> -- MatrixUtils.cpp:1307-1446, in two halves (the split only exposes the point where
    // both operands have reached target + 2; the operations and their order are those of the reference function).
    void ccmm_prepare(const CtT &op1, const CtT &op2, int target_level, Ct &sa, Ct &tb) {
        const i64 num_rows = op1.sh.rows, num_cols = op2.sh.cols;
        if (op1.sh.cols != op2.sh.rows) throw std::invalid_argument("[getCommonInsideLength] different inside length.");
        if (op1.sh.width != op2.sh.width) throw std::invalid_argument("[getCommonBlockWidth] different block width");
        const i64 width = op1.sh.width;
        i64 num_k = pow2_ceil(op1.sh.cols);
        if (std::min(op1.ct.level, op2.ct.level) < target_level + 3) throw std::invalid_argument("[multMatMat] level too low");
        CtT a = op1, b = op2;
        a.sh = Shape(num_rows, num_k, width); b.sh = Shape(num_k, num_cols, width);
        if (mode == 2) { // transforms at the lowest level that still leaves target + 2 (as multMatMatPre and the low-rank products do)
            a.ct = ev.level_down(a.ct, target_level + 3);
            b.ct = ev.level_down(b.ct, target_level + 3);
        }
        a = diagonal_to_column(a);
        b = diagonal_to_row(b);
        sa = ev.level_down(a.ct, target_level + 2);
        tb = ev.level_down(b.ct, target_level + 2);
    }
    CtT ccmm_core(Ct a, Ct b, i64 num_rows, i64 inner, i64 num_cols, i64 width, int target_level) {
        const i64 num_k = pow2_ceil(inner);
        if (a.level != target_level + 2 || b.level != target_level + 2) throw std::invalid_argument("[multMatMat] operands of the product loop must sit at target + 2");
        const Shape sha(num_rows, num_k, width), shb(num_k, num_cols, width);
        auto &col_mask = get_col_mask(sha, target_level + 2);
        auto &row_mask = get_row_mask(shb, target_level + 2);
        const i64 num_rows_tmp = (num_k > num_rows) ? num_k : pow2_ceil(num_rows);
        const i64 num_cols_tmp = (num_k > num_cols) ? num_k : pow2_ceil(num_cols);
        Ct res = ev.mul(a, b);
        Ct itxt_res;
        if (mode == 2) {
            for (i64 i = 1; i < num_k; i++) {
                ev.gen_rot_key(i); ev.gen_rot_key(i - num_cols_tmp); ev.gen_rot_key(i * width); ev.gen_rot_key((i - num_rows_tmp) * width);
                Ct tmp1 = ev.assemble_rot(a, i, col_mask[(size_t)(2 * i + 1)], i - num_cols_tmp, col_mask[(size_t)(2 * i)]);
                Ct tmp2 = ev.assemble_rot(b, i * width, row_mask[(size_t)(2 * i + 1)], (i - num_rows_tmp) * width, row_mask[(size_t)(2 * i)]);
                Ct t = ev.tensor(tmp1, tmp2);
                itxt_res = (i == 1) ? t : ev.add(itxt_res, t);
            }
        } else if (mode >= 1) {
            for (i64 i = 1; i < num_k; i++) {
                Ct tmp1 = assemble(rotL(a, i), col_mask[(size_t)(2 * i + 1)], rotL(a, i - num_cols_tmp), col_mask[(size_t)(2 * i)]);
                Ct tmp2 = assemble(rotL(b, i * width), row_mask[(size_t)(2 * i + 1)], rotL(b, (i - num_rows_tmp) * width), row_mask[(size_t)(2 * i)]);
                Ct t = ev.tensor(tmp1, tmp2);
                itxt_res = (i == 1) ? t : ev.add(itxt_res, t);
            }
        } else {
            a = rotL(a, 1);
            b = rotL(b, width);
            Ct a_rot = rotR(a, num_cols_tmp);
            Ct b_rot = rotR(b, num_rows_tmp * width);
            for (i64 i = 1; i < num_k; i++) {
                if (i > 1) {
                    a = rotL(a, 1); a_rot = rotL(a_rot, 1);
                    b = rotL(b, width); b_rot = rotL(b_rot, width);
                }
                Ct tmp1 = assemble(a, col_mask[(size_t)(2 * i + 1)], a_rot, col_mask[(size_t)(2 * i)]);
                Ct tmp2 = assemble(b, row_mask[(size_t)(2 * i + 1)], b_rot, row_mask[(size_t)(2 * i)]);
                Ct t = ev.tensor(tmp1, tmp2);
                itxt_res = (i == 1) ? t : ev.add(itxt_res, t);
            }
        }
        Ct tail = ev.rescale(ev.relin(itxt_res));
        res = ev.add(res, tail);
        return CtT{res, Shape(num_rows, num_cols, width)};
    }
    CtT mult_mat_mat_cc(const CtT &op1, const CtT &op2, int target_level) {
        Ct a, b;
        ccmm_prepare(op1, op2, target_level, a, b);
        return ccmm_core(std::move(a), std::move(b), op1.sh.rows, op1.sh.cols, op2.sh.cols, op1.sh.width, target_level);
    }

    // multPackedMatMat -- MatrixUtils.cpp:1100-1216
    CtT mult_packed_mat_mat(const CtT &op1, const CtT &op2, int target_level) {
        const i64 num_rows = op1.sh.rows, num_cols = op2.sh.cols;
        if (op1.sh.cols != op2.sh.rows) throw std::invalid_argument("[getCommonInsideLength] different inside length.");
        if (op1.sh.width != op2.sh.width) throw std::invalid_argument("[getCommonBlockWidth] different block width");
        const i64 width = op1.sh.width;
        i64 num_k = pow2_ceil(op1.sh.cols);
        if (op1.ct.level < target_level + 3 || op2.ct.level < target_level + 2) throw std::invalid_argument("[multMatMat] level too low");
        CtT a = op1, b = op2;
        a.sh = Shape(num_rows, num_k, width); b.sh = Shape(num_k, num_cols, width);
        auto &col_mask = get_col_mask(a.sh, target_level + 2);
        a.ct = ev.level_down(a.ct, target_level + 3);
        b.ct = ev.level_down(b.ct, target_level + 2);
        a = packed_diagonal_to_column(a);
        b = packed_diagonal_to_row(b);
        const i64 num_cols_tmp = (num_k > num_cols) ? num_k : pow2_ceil(num_cols);
        Ct res = ev.mul(a.ct, b.ct);
        Ct itxt_res;
        if (mode >= 1) {
            for (i64 i = 1; i < num_k / 2; i++) {
                Ct tmp1 = assemble(rotL(a.ct, 2 * i), col_mask[(size_t)(4 * i + 1)], rotL(a.ct, 2 * i - num_cols_tmp), col_mask[(size_t)(4 * i)]);
                Ct t = ev.tensor(tmp1, rotL(b.ct, 2 * i * width));
                itxt_res = (i == 1) ? t : ev.add(itxt_res, t);
            }
        } else {
            a.ct = rotL(a.ct, 2);
            b.ct = rotL(b.ct, 2 * width);
            Ct a_rot = rotR(a.ct, num_cols_tmp);
            for (i64 i = 1; i < num_k / 2; i++) {
                if (i > 1) {
                    a.ct = rotL(a.ct, 2); a_rot = rotL(a_rot, 2);
                    b.ct = rotL(b.ct, 2 * width);
                }
                Ct tmp1 = assemble(a.ct, col_mask[(size_t)(4 * i + 1)], a_rot, col_mask[(size_t)(4 * i)]);
                Ct t = ev.tensor(tmp1, b.ct);
                itxt_res = (i == 1) ? t : ev.add(itxt_res, t);
            }
        }
        Ct tail = ev.rescale(ev.relin(itxt_res));
        res = ev.add(res, tail);
        return CtT{res, Shape(num_rows, num_cols, width)};
    }
    // multPackedMatMatPre -- MatrixUtils.cpp:1218-1226
    CtT mult_packed_mat_mat_pre(const CtT &a_in, int target_level) {
        CtT a = a_in; a.ct = ev.level_down(a.ct, target_level + 3);
        return packed_diagonal_to_column(a);
    }
    // multPackedMatMatPreRot -- MatrixUtils.cpp:1228-1264.  Returns a batch of rows/2 ciphertexts.
    Ct mult_packed_mat_mat_pre_rot(const CtT &a_in, int target_level) {
        const i64 num_rows = a_in.sh.rows;
        std::vector<Ct> tmp;
        Ct a = a_in.ct;
        tmp.push_back(ev.level_down(a, a.level - 1));
        auto &col_mask = get_col_mask(a_in.sh, target_level + 2);
        if (mode >= 1) {
            for (i64 i = 1; i < num_rows / 2; i++)
                tmp.push_back(assemble(rotL(a_in.ct, 2 * i), col_mask[(size_t)(4 * i + 1)], rotL(a_in.ct, 2 * i - num_rows), col_mask[(size_t)(4 * i)]));
            return stack(tmp);
        }
        a = rotL(a, 2);
        Ct a_rot = rotR(a, num_rows);
        for (i64 i = 1; i < num_rows / 2; i++) {
            if (i > 1) { a = rotL(a, 2); a_rot = rotL(a_rot, 2); }
            tmp.push_back(assemble(a, col_mask[(size_t)(4 * i + 1)], a_rot, col_mask[(size_t)(4 * i)]));
        }
        return stack(tmp);
    }
    // multPackedMatMatPreRev -- MatrixUtils.cpp:1266-1274
    CtT mult_packed_mat_mat_pre_rev(const CtT &b_in, int target_level) {
        CtT b = b_in; b.ct = ev.level_down(b.ct, target_level + 2);
        return packed_diagonal_to_row(b);
    }
    // multPackedMatMatCCReuse -- MatrixUtils.cpp:1276-1305 (relinearised and rescaled)
    CtT mult_packed_mat_mat_cc_reuse(const Ct &pre, const CtT &b_in) {
        const i64 width = b_in.sh.width;
        Ct b = b_in.ct;
        Ct sum = ev.tensor(slice(pre, 0), b);
        for (int i = 1; i < pre.batch; ++i) {
            b = mode >= 1 ? rotL(b_in.ct, (i64)i * 2 * width) : rotL(b, 2 * width);
            sum = ev.add(sum, ev.tensor(slice(pre, i), b));
        }
        return CtT{ev.rescale(ev.relin(sum)), Shape(b_in.sh.rows, b_in.sh.cols, width)};
    }

    // multMatMatPre -- MatrixUtils.cpp:1572-1610.  Returns the `rows` shifted copies as one batch.
    Ct mult_mat_mat_pre(const CtT &a_in, int target_level) {
        const i64 num_rows = a_in.sh.rows;
        CtT a = a_in;
        a.ct = ev.level_down(a.ct, target_level + 3);
        a = diagonal_to_column(a);
        std::vector<Ct> tmp;
        tmp.push_back(ev.level_down(a.ct, a.ct.level - 1));
        auto &col_mask = get_col_mask(a.sh, target_level + 2);
        if (mode == 2) {
            for (i64 i = 1; i < num_rows; i++) {
                ev.gen_rot_key(i); ev.gen_rot_key(i - num_rows);
                tmp.push_back(ev.assemble_rot(a.ct, i, col_mask[(size_t)(2 * i + 1)], i - num_rows, col_mask[(size_t)(2 * i)]));
            }
            return stack(tmp);
        }
        if (mode >= 1) {
            for (i64 i = 1; i < num_rows; i++)
                tmp.push_back(assemble(rotL(a.ct, i), col_mask[(size_t)(2 * i + 1)], rotL(a.ct, i - num_rows), col_mask[(size_t)(2 * i)]));
            return stack(tmp);
        }
        a.ct = rotL(a.ct, 1);
        Ct a_rot = rotR(a.ct, num_rows);
        for (i64 i = 1; i < num_rows; i++) {
            if (i > 1) { a.ct = rotL(a.ct, 1); a_rot = rotL(a_rot, 1); }
            tmp.push_back(assemble(a.ct, col_mask[(size_t)(2 * i + 1)], a_rot, col_mask[(size_t)(2 * i)]));
        }
        return stack(tmp);
    }
    // multMatMatReUse -- MatrixUtils.cpp:1612-1639 with HomEvaluator::matmul (HomEvaluator.hpp:595-601):
    //   out = sum_k pre[k] (.) leftRotate(pt, k * width), un-rescaled (scale Delta^2).
    // The plaintext must already sit at the level of `pre` (the reference re-encodes otherwise).
    CtT mult_mat_mat_reuse(const Ct &pre, const PtT &b) {
        if (b.pt.level != pre.level) throw std::invalid_argument("[multMatMatReUse] plaintext level differs from the ciphertexts'");
        Ct acc;
        for (int k = 0; k < pre.batch; ++k) {
            Pt pk = pt_rotate(b.pt, (i64)k * b.sh.width);
            Ct t = ev.mul_pt_norescale(slice(pre, k), pk);
            acc = (k == 0) ? t : ev.add(acc, t);
        }
        return CtT{acc, Shape(b.sh.rows, b.sh.cols, b.sh.width)};
    }
    // multMatMatPreRev -- MatrixUtils.cpp:1641-1649
    CtT mult_mat_mat_pre_rev(const CtT &b_in, int target_level) {
        CtT b = b_in; b.ct = ev.level_down(b.ct, target_level + 2);
        return diagonal_to_row(b);
    }
    // multMatMatCCReUse -- MatrixUtils.cpp:1651-1679 (relinearised, NOT rescaled)
    CtT mult_mat_mat_cc_reuse(const Ct &pre, const CtT &b_in) {
        const i64 width = b_in.sh.width;
        Ct b = b_in.ct;
        Ct sum = ev.tensor(slice(pre, 0), b);
        for (int i = 1; i < pre.batch; ++i) {
            b = mode >= 1 ? rotL(b_in.ct, (i64)i * width) : rotL(b, width);
            sum = ev.add(sum, ev.tensor(slice(pre, i), b));
        }
        return CtT{ev.relin(sum), Shape(b_in.sh.rows, b_in.sh.cols, width)};
    }

    // Plaintext arithmetic used by multMatMat<Plaintext>: a plaintext is a one-polynomial ciphertext without key material,
    // so product (with rescale) and sum are the ciphertext operations on one polynomial.
    static Ct pt_as_ct(const Pt &p) { Ct c(p.N, p.level, 1, 1, p.spow, p.d.empty()); c.d = p.d; return c; }
    static Pt ct_as_pt(const Ct &c) { Pt p; p.level = c.level; p.spow = c.spow; p.N = c.N; p.d = c.d; return p; }
    Pt pt_mul(const Pt &a, const Pt &b) { return ct_as_pt(ev.rescale(ev.mul_pt_norescale(pt_as_ct(a), b))); }
    Pt pt_add(const Pt &a, const Pt &b) { return ct_as_pt(ev.add(pt_as_ct(a), pt_as_ct(b))); }

    // multMatMat<Plaintext> -- MatrixUtils.cpp:1448-1570 (HEMMer::singleMatMul), with the cleartext tau of
    // diagonalToRow<Plaintext> (:1072-1098).  `msg` is the decoded right operand (the reference decodes the Plaintext).
    CtT mult_mat_mat_cp(const CtT &op1, const Message &msg, const Shape &shb, int target_level) {
        const i64 num_rows = op1.sh.rows, num_cols = shb.cols, width = op1.sh.width;
        if (op1.sh.cols != shb.rows) throw std::invalid_argument("[getCommonInsideLength] different inside length.");
        if (width != shb.width) throw std::invalid_argument("[getCommonBlockWidth] different block width");
        const i64 num_k = pow2_ceil(op1.sh.cols);
        if (op1.ct.level < target_level + 3) throw std::invalid_argument("[multMatMat] level too low");
        CtT a = op1; a.sh = Shape(num_rows, num_k, width);
        const Shape sb(num_k, num_cols, width);
        a = diagonal_to_column(a);
        Message m2((size_t)slots, cplx(0, 0));
        for (i64 i = 0; i < sb.rows; i++)
            for (i64 j = 0; j < sb.cols; j++) {
                m2[(size_t)(((i - j + sb.rows) % sb.rows) * width + j)] = msg[(size_t)(i * width + j)];
                if (width != sb.cols) m2[(size_t)(((i - j + sb.rows) % sb.rows) * width + sb.cols + j)] = msg[(size_t)(i * width + j + sb.cols)];
            }
        a.ct = ev.level_down(a.ct, target_level + 2);
        Pt b = ev.encode(m2.data(), m2.size(), target_level + 2);
        const i64 num_rows_tmp = (num_k > num_rows) ? num_k : pow2_ceil(num_rows);
        const i64 num_cols_tmp = (num_k > num_cols) ? num_k : pow2_ceil(num_cols);
        Ct res = ev.mul_pt(a.ct, b);
        a.ct = rotL(a.ct, 1);
        b = pt_rotate(b, width);
        Ct a_rot = rotR(a.ct, num_cols_tmp);
        Pt b_rot = pt_rotate(b, -num_rows_tmp * width);
        auto &col_mask = get_col_mask(a.sh, target_level + 2);
        auto &row_mask = get_row_mask(sb, target_level + 2);
        Ct itxt_res;
        for (i64 i = 1; i < num_k; i++) {
            if (i > 1) {
                a.ct = rotL(a.ct, 1); a_rot = rotL(a_rot, 1);
                b = pt_rotate(b, width); b_rot = pt_rotate(b_rot, width);
            }
            Ct tmp1 = assemble(a.ct, col_mask[(size_t)(2 * i + 1)], a_rot, col_mask[(size_t)(2 * i)]);
            Pt tmp3 = pt_add(pt_mul(b, row_mask[(size_t)(2 * i + 1)]), pt_mul(b_rot, row_mask[(size_t)(2 * i)]));
            Ct t = ev.mul_pt(tmp1, tmp3);
            itxt_res = (i == 1) ? t : ev.add(itxt_res, t);
        }
        res = ev.add(res, itxt_res);
        return CtT{res, Shape(num_rows, num_cols, width)};
    }

    // leftRotate on a plaintext: the slot permutation alone (no key), used by HomEvaluator::matmul
    Pt pt_rotate(const Pt &p, i64 left_steps) {
        u64 g = cx.galois_for_rotation(left_steps);
        if (g == 1 || ev.dry) return p;
        const auto &perm = cx.ntt_perm(g);
        Pt r = p;
        for (int l = 0; l <= p.level; ++l)
            for (int c = 0; c < cx.N; ++c) r.limb(l)[c] = p.limb(l)[perm[(size_t)c]];
        return r;
    }
    Ct slice(const Ct &b, int k) const {
        if (ev.dry) return ev.meta(b.level, b.np, 1, b.spow);
        Ct r(cx.N, b.level, b.np, 1, b.spow);
        std::memcpy(r.d.data(), b.limb(k, 0, 0), r.d.size() * 8);
        return r;
    }
    // copy k of input b lands at batch position k * B + b (B = batch of each element)
    Ct stack(const std::vector<Ct> &v) const {
        const int B = v[0].batch;
        if (ev.dry) return ev.meta(v[0].level, v[0].np, (int)v.size() * B, v[0].spow);
        Ct r(cx.N, v[0].level, v[0].np, (int)v.size() * B, v[0].spow);
        for (size_t k = 0; k < v.size(); ++k) {
            if (v[k].level != r.level || v[k].np != r.np || v[k].batch != B) throw std::invalid_argument("stack: mismatched ciphertexts");
            std::memcpy(r.limb((int)k * B, 0, 0), v[k].d.data(), v[k].d.size() * 8);
        }
        return r;
    }
    // matMulReUse summed over K-groups (addInplace over groups, bert-matmul.cpp:262-268)
    CtT mult_mat_mat_reuse_groups(const Ct &pre, int btotal, int b0, const std::vector<const Pt *> &pts, i64 width) {
        const int kc = pre.batch / btotal;
        Ct acc;
        bool first = true;
        for (size_t b = 0; b < pts.size(); ++b)
            for (int k = 0; k < kc; ++k) {
                if (pts[b]->level != pre.level) throw std::invalid_argument("[multMatMatReUse] plaintext level differs from the ciphertexts'");
                Ct t = ev.mul_pt_norescale(slice(pre, k * btotal + b0 + (int)b), pt_rotate(*pts[b], (i64)k * width));
                acc = first ? t : ev.add(acc, t);
                first = false;
            }
        return CtT{acc, Shape()};
    }

    // ---------------- HEMMer-level helpers ----------------
    // generateAxisMasks / generateRightLeftMasks -- HEMMer.cpp:2345-2393, two tiles side by side
    void gen_axis_masks() {
        const i64 d = tile;
        col_mask_even_.msg.assign((size_t)slots, cplx(0, 0));
        row_mask_even_.msg.assign((size_t)slots, cplx(0, 0));
        mask_left_half_.msg.assign((size_t)slots, cplx(0, 0));
        if (2 * d * d != slots) return; // slot count not of the form 2*d^2: HEMMer-level packing unavailable
        for (i64 r = 0; r < d; ++r)
            for (i64 c = 0; c < 2 * d; ++c) {
                size_t s = (size_t)(r * 2 * d + c);
                if ((c % d) % 2 == 0) col_mask_even_.msg[s] = 1;
                if (r % 2 == 0) row_mask_even_.msg[s] = 1;
                if (c < d) mask_left_half_.msg[s] = 1;
            }
    }
    // mask_matmul_ = encode2(one, zero) -- HEMMer.cpp:2336-2339 (a Plaintext at the operand's level)
    const Pt &mask_matmul(int level) {
        auto it = mask_matmul_.find(level);
        if (it == mask_matmul_.end()) it = mask_matmul_.emplace(level, ev.encode(mask_left_half_.msg.data(), (size_t)slots, level)).first;
        return it->second;
    }
    // complexPackingInplace -- HEMMer.cpp:764-777
    void complex_packing_inplace(CtT &t) {
        Ct even = mult_msg(t.ct, col_mask_even_);
        Ct odd = rotL(t.ct, 1);
        odd = ev.mult_imag(odd);
        odd = mult_msg(odd, col_mask_even_);
        Ct fus = ev.add(odd, even);
        t.ct = rotR(fus, 1);
        t.ct = ev.add(t.ct, fus);
    }
    // transposeInplace -- HEMMer.cpp:1166-1172
    void transpose_inplace(CtT &t, int target_level) {
        if (target_level > 0) t.ct = ev.level_down(t.ct, 1 + target_level);
        t = transpose(t);
    }
    // transposeComplexPackingInplace -- HEMMer.cpp:779-799
    void transpose_complex_packing_inplace(CtT &t, int target_level) {
        Ct even = mult_msg(t.ct, col_mask_even_);
        Ct odd = rotL(t.ct, 1);
        odd = ev.mult_imag(odd);
        odd = ev.negate(odd);
        odd = mult_msg(odd, col_mask_even_);
        Ct fus = ev.add(odd, even);
        t.ct = rotR(fus, 1);
        t.ct = ev.add(t.ct, fus);
        if (target_level > 0) t.ct = ev.level_down(t.ct, 1 + target_level);
        transpose_inplace(t, 0);
    }
    // complexPackingRowInplace -- HEMMer.cpp:801-817
    void complex_packing_row_inplace(CtT &t) {
        const i64 bw = t.sh.width;
        Ct even = mult_msg(t.ct, row_mask_even_);
        Ct odd = rotL(t.ct, bw);
        odd = ev.mult_imag(odd);
        odd = ev.negate(odd);
        odd = mult_msg(odd, row_mask_even_);
        Ct fus = ev.add(even, odd);
        t.ct = rotR(fus, bw);
        t.ct = ev.add(t.ct, fus);
    }
    // splitInTwo -- HEMMer.cpp:819-831
    void split_in_two(const CtT &t, CtT &t1, CtT &t2) {
        const i64 width = t.sh.cols;
        Ct tmp = mult_msg(t.ct, mask_left_half_);
        t1.sh = t2.sh = t.sh;
        t2.ct = ev.add(t.ct, tmp, true);
        t1.ct = rotR(tmp, width);
        t1.ct = ev.add(t1.ct, tmp);
        Ct tmp2 = rotL(t2.ct, width);
        t2.ct = ev.add(t2.ct, tmp2);
    }
    // oneMatRotSumInplace -- HEMMer.cpp:882-919, ModelArgs::HEAD_DIM = tile side: the row sums of the left halves of the
    // tiles of a (first column) and of the right halves of the tiles of b (last column), spread over the whole row
    void one_mat_rot_sum_inplace(CtT &a, CtT &b) {
        const i64 d = tile;
        for (i64 rot = 1; rot < d / 2; rot <<= 1) {
            a.ct = ev.add(a.ct, rotL(a.ct, rot));
            b.ct = ev.add(b.ct, rotR(b.ct, rot));
        }
        Mask first, last;
        first.msg.assign((size_t)slots, cplx(0, 0));
        last.msg.assign((size_t)slots, cplx(0, 0));
        for (i64 r = 0; r < d; ++r)
            for (i64 t = 0; t < 2; ++t) {
                first.msg[(size_t)(r * 2 * d + t * d)] = 1;
                last.msg[(size_t)(r * 2 * d + t * d + d - 1)] = 1;
            }
        a.ct = mult_msg(a.ct, first);
        b.ct = mult_msg(b.ct, last);
        for (i64 rot = 1; rot < d; rot <<= 1) {
            a.ct = ev.add(a.ct, rotR(a.ct, rot));
            b.ct = ev.add(b.ct, rotL(b.ct, rot));
        }
    }
    // HEMMer::maskFirstColInplace / maskLeftHalfInplace / maskRightHalfInplace -- HEMMer.cpp:1251-1269
    Ct mask_inplace(const Ct &x, int which) {
        const i64 d = tile;
        Mask m;
        m.msg.assign((size_t)slots, cplx(0, 0));
        for (i64 r = 0; r < d; ++r)
            for (i64 c = 0; c < 2 * d; ++c)
                if (which == 0 ? (c % d == 0) : which == 1 ? (c < d) : (c >= d)) m.msg[(size_t)(r * 2 * d + c)] = 1;
        return mult_msg(x, m);
    }
    // HEMMer::squareSum -- HEMMer.cpp:2499-2510
    Ct square_sum(const std::vector<Ct> &v) {
        Ct acc = ev.tensor(v[0], v[0]);
        for (size_t i = 1; i < v.size(); ++i) acc = ev.add(acc, ev.tensor(v[i], v[i]));
        return ev.rescale(ev.relin(acc));
    }
    // HEMMer::reduceRowSumWithScaledMask -- HEMMer.cpp:2512-2530, one rank
    Ct reduce_row_sum_with_scaled_mask(Ct x, const Pt &mask, i64 width) {
        for (i64 i = 1; i < width; i <<= 1) x = ev.add(x, rotL(x, i));
        x = ev.mul_pt(x, mask);
        for (i64 i = 1; i < width; i <<= 1) x = ev.add(x, rotR(x, i));
        return x;
    }
    // HEMMer::tr_oneMatRotSumInplace -- HEMMer.cpp:921-962 (HEAD_DIM = tile side)
    void tr_one_mat_rot_sum_inplace(CtT &a, CtT &b, int target_level) {
        const i64 d = tile;
        if (target_level > 0) {
            a.ct = ev.level_down(a.ct, target_level + 1);
            b.ct = ev.level_down(b.ct, target_level + 1);
        }
        for (i64 rot = 1; rot < d; rot <<= 1) {
            a.ct = ev.add(a.ct, rotL(a.ct, rot));
            b.ct = ev.add(b.ct, rotR(b.ct, rot));
        }
        Mask first, last;
        first.msg.assign((size_t)slots, cplx(0, 0));
        last.msg.assign((size_t)slots, cplx(0, 0));
        for (i64 r = 0; r < d; ++r)
            for (i64 t = 0; t < 2; ++t) {
                first.msg[(size_t)(r * 2 * d + t * d)] = 1;
                last.msg[(size_t)(r * 2 * d + t * d + d - 1)] = 1;
            }
        a.ct = mult_msg(a.ct, first);
        b.ct = mult_msg(b.ct, last);
        for (i64 rot = 1; rot < d / 2; rot <<= 1) {
            a.ct = ev.add(a.ct, rotR(a.ct, rot));
            b.ct = ev.add(b.ct, rotL(b.ct, rot));
        }
    }
    // Gaussian-kernel score assembly of attention2_bert_loraOpti -- TransformerBlock.cpp:2420-2482 (one query / key pair)
    std::vector<CtT> gaussian_kernel_scores(const CtT &query, const CtT &key, int target_level) {
        const i64 d = tile;
        Mask left, right;
        left.msg.assign((size_t)slots, cplx(0, 0));
        right.msg.assign((size_t)slots, cplx(0, 0));
        for (i64 r = 0; r < d; ++r)
            for (i64 c = 0; c < 2 * d; ++c) ((c % d) < d / 2 ? left : right).msg[(size_t)(r * 2 * d + c)] = 1;
        std::vector<CtT> mq{CtT{mult_msg(query.ct, left), query.sh}, CtT{mult_msg(query.ct, right), query.sh}};
        std::vector<CtT> mk{CtT{mult_msg(key.ct, left), key.sh}, CtT{mult_msg(key.ct, right), key.sh}};
        std::vector<CtT> oq, ok;
        for (int j = 0; j < 2; ++j) {
            oq.push_back(CtT{ev.mul(mq[(size_t)j].ct, mq[(size_t)j].ct), query.sh});
            ok.push_back(CtT{ev.mul(mk[(size_t)j].ct, mk[(size_t)j].ct), key.sh});
        }
        one_mat_rot_sum_inplace(oq[0], oq[1]);
        one_mat_rot_sum_inplace(ok[0], ok[1]);
        for (auto &t : ok) transpose_inplace(t, target_level);
        std::vector<CtT> out;
        for (size_t j = 0; j < 2; ++j) {
            complex_packing_inplace(mq[j]);
            transpose_inplace(mk[j], 0);
            complex_packing_row_inplace(mk[j]);
            CtT s = repack_cc(mult_packed_mat_mat(mq[j], mk[j], target_level));
            s.ct = ev.mult_int(s.ct, -2);
            s.ct = ev.add(s.ct, oq[j].ct);
            s.ct = ev.add(s.ct, ok[j].ct);
            out.push_back(std::move(s));
        }
        return out;
    }
    // the rank-2 LoRA branch of attention2_bert_loraOpti -- TransformerBlock.cpp:2199-2365 (without the bootstraps)
    std::vector<Ct> lora_opti_forward(const std::vector<Ct> &cur, const Ct &lora_wa, const Ct &lora_wb) {
        const i64 d = tile, w = 2 * tile;
        Mask first_row, first_col_only;
        first_row.msg.assign((size_t)slots, cplx(0, 0));
        first_col_only.msg.assign((size_t)slots, cplx(0, 0));
        for (i64 c = 0; c < w; ++c) first_row.msg[(size_t)c] = 1;
        for (i64 r = 0; r < d; ++r) first_col_only.msg[(size_t)(r * w)] = 1;
        auto rank_rows = [&](const Ct &factor) {
            std::vector<std::vector<Ct>> rows;
            for (i64 i = 0; i < 3; ++i) {
                Ct base = i == 0 ? factor : rotL(factor, i * 2 * w);
                std::vector<Ct> pair{base, rotL(base, w)};
                for (auto &t : pair) {
                    t = mult_msg(t, first_row);
                    for (i64 rot = 1; rot < d; rot <<= 1) t = ev.add(t, rotR(t, rot * w));
                }
                rows.push_back(std::move(pair));
            }
            return rows;
        };
        const auto wa = rank_rows(lora_wa);
        std::vector<Ct> xa;
        for (int j = 0; j < 2; ++j) {
            Ct acc = ev.mul(cur[0], wa[0][(size_t)j]);
            for (size_t i = 1; i < 3; ++i) acc = ev.add(acc, ev.mul(cur[i], wa[i][(size_t)j]));
            for (i64 rot = 1; rot < w; rot <<= 1) acc = ev.add(acc, rotL(acc, rot));
            xa.push_back(mult_msg(acc, first_col_only));
        }
        const auto wb = rank_rows(lora_wb);
        for (auto &t : xa)
            for (i64 rot = 1; rot < w; rot <<= 1) t = ev.add(t, rotR(t, rot));
        std::vector<Ct> out;
        for (size_t i = 0; i < 3; ++i) out.push_back(ev.add(ev.mul(xa[0], wb[i][0]), ev.mul(xa[1], wb[i][1])));
        return out;
    }
    // repackCC -- HEMMer.cpp:964-969
    CtT repack_cc(const CtT &t) {
        ev.gen_galois_key(cx.galois_conj());
        return CtT{ev.add(t.ct, ev.conjugate(t.ct)), t.sh};
    }
    // complexPacking(ct, ct) -- HEMMer.cpp:980-986 ; complexPackingRev -- :988-994
    CtT complex_packing(const CtT &a, const CtT &b) { return CtT{ev.add(a.ct, ev.mult_imag(b.ct)), b.sh}; }
    CtT complex_packing_rev(const CtT &a, const CtT &b) { return CtT{ev.add(a.ct, ev.mult_imag(b.ct), true), b.sh}; }
    // repack_notBTS -- HEMMer.cpp:1025-1053
    CtT repack_not_bts(const CtT &t1, const CtT &t2) {
        Ct a = ev.rescale(t1.ct), b = ev.rescale(t2.ct);
        Ct out = ev.add(a, ev.conjugate(a));
        Ct tmp = ev.add(b, ev.conjugate(b));
        tmp = ev.mult_imag(tmp);
        out = ev.add(out, tmp);
        tmp = rotL(out, tile);
        out = ev.add(out, tmp);
        tmp = ev.mul_pt(tmp, mask_matmul(tmp.level));
        out = ev.mul_pt(out, mask_matmul(out.level));
        tmp = rotR(tmp, tile);
        out = ev.add(out, tmp);
        return CtT{out, t1.sh};
    }
    // repack_loraOpti -- HEMMer.cpp:1055-1091 (mask_matmul_half_ = encode2(0.5, 0), HEMMer.cpp:2341-2342)
    Mask mask_left_half_scaled_;
    CtT repack_lora_opti(const CtT &t1, const CtT &t2) {
        if (mask_left_half_scaled_.msg.empty()) {
            mask_left_half_scaled_.msg = mask_left_half_.msg;
            for (auto &v : mask_left_half_scaled_.msg) v *= 0.5;
        }
        ev.gen_galois_key(cx.galois_conj());
        Ct a = ev.rescale(t1.ct), b = ev.rescale(t2.ct);
        Ct out = ev.add(a, ev.conjugate(a));
        Ct tmp = ev.add(b, ev.conjugate(b));
        tmp = ev.mult_imag(tmp);
        out = ev.add(out, tmp);
        tmp = rotL(out, tile);
        out = ev.add(out, tmp);
        Ct conj_tmp = ev.conjugate(out);
        out = ev.add(out, conj_tmp);
        tmp = ev.add(conj_tmp, tmp, true);
        tmp = ev.mult_imag(tmp);
        tmp = mult_msg(tmp, mask_left_half_scaled_);
        out = mult_msg(out, mask_left_half_scaled_);
        tmp = rotR(tmp, tile);
        out = ev.add(out, tmp);
        return CtT{out, t1.sh};
    }

    // ---------------- LoRA low-rank products ----------------
    // A thin factor (low_dim columns or rows) needs only low_dim terms of the product loop; the remaining terms
    // of the inner sum are folded by the log-step rotate-and-add trees below and in the repackTo* helpers.
    // low_dim is ModelArgs::LOW_DIM in the reference (ModelArgs.hpp:67); here it is an argument.
    std::map<std::tuple<int, Shape, i64, i64>, Mask> low_mask_;
    Mask &low_mask(int kind, const Shape &s, i64 block, i64 low_dim) { return low_mask_[std::make_tuple(kind, s, block, low_dim)]; }

    // the k = 0 term and the low_dim - 1 shifted terms -- shared tail of MatrixUtils.cpp:1716-1768, 1809-1876, 1929-1996
    CtT low_rank_tail(Ct a, Ct b, const Shape &sh1, const Shape &sh2, i64 width, i64 low_dim, int target_level) {
        const i64 num_rows = sh1.rows;
        Ct res = ev.mul(a, b);
        a = rotL(a, 1);
        b = rotL(b, width);
        Ct a_rot = rotR(a, width / 2);
        Ct b_rot = rotR(b, num_rows * width);
        auto &col_mask = get_col_mask(sh1, target_level + 2);
        auto &row_mask = get_row_mask(sh2, target_level + 2);
        Ct itxt_res;
        for (i64 i = 1; i < low_dim; i++) {
            if (i > 1) {
                a = rotL(a, 1); a_rot = rotL(a_rot, 1);
                b = rotL(b, width); b_rot = rotL(b_rot, width);
            }
            Ct tmp1 = assemble(a, col_mask[(size_t)(2 * i + 1)], a_rot, col_mask[(size_t)(2 * i)]);
            Ct tmp2 = assemble(b, row_mask[(size_t)(2 * i + 1)], b_rot, row_mask[(size_t)(2 * i)]);
            Ct t = ev.tensor(tmp1, tmp2);
            itxt_res = (i == 1) ? t : ev.add(itxt_res, t);
        }
        if (low_dim > 1) res = ev.add(res, ev.rescale(ev.relin(itxt_res)));
        return CtT{res, Shape(sh1.rows, sh2.cols, sh2.width)};
    }
    void low_rank_check(const CtT &op1, const CtT &op2, int target_level, i64 low_dim) {
        if (low_dim < 1 || (low_dim & (low_dim - 1))) throw std::invalid_argument("[lowRank] low_dim must be a power of two");
        if (std::min(op1.ct.level, op2.ct.level) < target_level + 3) throw std::invalid_argument("[lowRank] level too low");
    }
    // multMatMatHighLow -- MatrixUtils.cpp:1681-1771
    CtT mult_mat_mat_high_low(const CtT &op1, const CtT &op2, i64 in_col_block, int target_level, i64 low_dim) {
        low_rank_check(op1, op2, target_level, low_dim);
        const i64 width = op2.sh.width;
        CtT a = op1, b = op2;
        b.sh = Shape(op2.sh.rows, low_dim, op2.sh.width);
        a.ct = ev.level_down(a.ct, target_level + 3);
        b.ct = ev.level_down(b.ct, target_level + 3);
        a = diagonal_to_column(a);
        b = diagonal_to_row(b);
        i64 col_pos = in_col_block;
        for (i64 i = low_dim; i < width / 2; i <<= 1) {
            Ct tmp;
            if (col_pos % 2 == 0) {
                tmp = rotL(b.ct, i * width);
                tmp = rotR(tmp, i);
            } else {
                tmp = rotL(b.ct, i);
                b.ct = rotL(b.ct, i * width);
            }
            b.ct = ev.add(b.ct, tmp);
            col_pos /= 2;
        }
        return low_rank_tail(a.ct, b.ct, op1.sh, op2.sh, width, low_dim, target_level);
    }
    // multMatMatLowHigh -- MatrixUtils.cpp:1773-1879
    CtT mult_mat_mat_low_high(const CtT &op1, const CtT &op2, i64 in_row_block, int target_level, i64 low_dim) {
        low_rank_check(op1, op2, target_level, low_dim);
        if (op1.sh.width != op2.sh.width) throw std::invalid_argument("[getCommonBlockWidth] different block width");
        const i64 width = op1.sh.width;
        CtT a = op1, b = op2;
        a.ct = ev.level_down(a.ct, target_level + 3);
        b.ct = ev.level_down(b.ct, target_level + 3);
        i64 row_pos = in_row_block;
        for (i64 i = low_dim; i < width / 2; i <<= 1) {
            Ct tmp = (row_pos % 2 == 0) ? rotR(a.ct, i * width) : rotL(a.ct, i * width);
            a.ct = ev.add(a.ct, tmp);
            row_pos /= 2;
        }
        a = diagonal_to_column(a);
        b = diagonal_to_row(b);
        return low_rank_tail(a.ct, b.ct, op1.sh, op2.sh, width, low_dim, target_level);
    }
    // multMatMatLowLow -- MatrixUtils.cpp:1881-1996
    CtT mult_mat_mat_low_low(const CtT &op1, const CtT &op2, i64 in_col_block, i64 in_row_block, int target_level, i64 low_dim) {
        low_rank_check(op1, op2, target_level, low_dim);
        if (op1.sh.width != op2.sh.width) throw std::invalid_argument("[getCommonBlockWidth] different block width");
        const i64 width = op1.sh.width;
        CtT a = op1, b = op2;
        a.sh = Shape(op1.sh.rows, low_dim, op1.sh.width);
        b.sh = Shape(low_dim, op2.sh.cols, op2.sh.width);
        a.ct = ev.level_down(a.ct, target_level + 3);
        b.ct = ev.level_down(b.ct, target_level + 3);
        a = diagonal_to_column(a);
        b = diagonal_to_row(b);
        i64 col_pos = in_col_block, row_pos = in_row_block;
        for (i64 i = low_dim; i < width / 2; i <<= 1) {
            Ct tmp = (col_pos % 2 == 0) ? rotR(a.ct, i) : rotL(a.ct, i);
            a.ct = ev.add(a.ct, tmp);
            col_pos /= 2;
            tmp = (row_pos % 2 == 0) ? rotR(b.ct, i * width) : rotL(b.ct, i * width);
            b.ct = ev.add(b.ct, tmp);
            row_pos /= 2;
        }
        return low_rank_tail(a.ct, b.ct, op1.sh, op2.sh, width, low_dim, target_level);
    }
    // repackToOneCol -- HEMMer.cpp:2131-2172
    CtT repack_to_one_col(const CtT &t, i64 out_col_block, i64 low_dim) {
        const i64 num_rows = t.sh.rows, num_cols = t.sh.cols, width = t.sh.width;
        CtT ret = t;
        i64 col_pos = out_col_block;
        for (i64 i = low_dim; i < width; i <<= 1) {
            Ct tmp = (col_pos % 2 == 0) ? rotL(ret.ct, i) : rotR(ret.ct, i);
            ret.ct = ev.add(ret.ct, tmp);
            col_pos /= 2;
        }
        Mask &m = low_mask(0, t.sh, out_col_block, low_dim);
        if (m.msg.empty()) {
            m.msg.assign((size_t)slots, cplx(0, 0));
            for (i64 i = 0; i < num_rows; i++)
                for (i64 j = out_col_block * low_dim; j < (1 + out_col_block) * low_dim; j++) m.msg[(size_t)(i * width + j)] = 1;
        }
        ret.ct = mult_msg(ret.ct, m);
        for (i64 i = num_cols; i < width; i <<= 1) ret.ct = ev.add(ret.ct, rotR(ret.ct, num_cols));
        return ret;
    }
    // repackToMultiCol -- HEMMer.cpp:2174-2209
    CtT repack_to_multi_col(const CtT &t, i64 out_col_block, i64 low_dim) {
        const i64 num_rows = t.sh.rows, num_cols = t.sh.cols, width = t.sh.width;
        CtT ret = t;
        i64 col_pos = out_col_block;
        for (i64 i = low_dim; i < width / 2; i <<= 1) {
            Ct tmp = (col_pos % 2 == 0) ? rotL(ret.ct, i) : rotR(ret.ct, i);
            ret.ct = ev.add(ret.ct, tmp);
            col_pos /= 2;
        }
        ret.ct = mult_msg(ret.ct, low_col_block_mask(t.sh, out_col_block, low_dim));
        (void)num_rows; (void)num_cols;
        return ret;
    }
    // repackToOneRow -- HEMMer.cpp:2211-2255
    CtT repack_to_one_row(const CtT &t, i64 out_row_block, i64 low_dim) {
        const i64 num_rows = t.sh.rows, num_cols = t.sh.cols, width = t.sh.width;
        CtT ret = t;
        i64 row_pos = out_row_block;
        for (i64 i = low_dim; i < num_rows; i <<= 1) {
            Ct tmp = (row_pos % 2 == 0) ? rotL(ret.ct, i * width) : rotR(ret.ct, i * width);
            ret.ct = ev.add(ret.ct, tmp);
            row_pos /= 2;
        }
        for (i64 i = num_cols; i < width; i <<= 1) ret.ct = ev.add(ret.ct, rotL(ret.ct, num_cols));
        Mask &m = low_mask(1, t.sh, out_row_block, low_dim);
        if (m.msg.empty()) {
            m.msg.assign((size_t)slots, cplx(0, 0));
            for (i64 i = out_row_block * low_dim; i < (1 + out_row_block) * low_dim; ++i)
                for (i64 j = 0; j < num_cols; j++) m.msg[(size_t)(i * width + j)] = 1;
        }
        ret.ct = mult_msg(ret.ct, m);
        for (i64 i = num_cols; i < width; i += num_cols) ret.ct = ev.add(ret.ct, rotR(ret.ct, num_cols));
        return ret;
    }
    // repackToMultiRow -- HEMMer.cpp:2257-2290
    CtT repack_to_multi_row(const CtT &t, i64 out_row_block, i64 low_dim) {
        const i64 num_rows = t.sh.rows, width = t.sh.width;
        CtT ret = t;
        i64 row_pos = out_row_block;
        for (i64 i = low_dim; i < num_rows; i <<= 1) {
            Ct tmp = (row_pos % 2 == 0) ? rotL(ret.ct, i * width) : rotR(ret.ct, i * width);
            ret.ct = ev.add(ret.ct, tmp);
            row_pos /= 2;
        }
        Mask &m = low_mask(2, t.sh, out_row_block, low_dim);
        if (m.msg.empty()) {
            m.msg.assign((size_t)slots, cplx(0, 0));
            for (i64 i = out_row_block * low_dim; i < (1 + out_row_block) * low_dim; ++i)
                for (i64 j = 0; j < width; j++) m.msg[(size_t)(i * width + j)] = 1;
        }
        ret.ct = mult_msg(ret.ct, m);
        return ret;
    }
    // the mask of getLowColBlock and repackToMultiCol: columns [block*low_dim, (block+1)*low_dim) of every
    // num_cols-wide tile of the first num_rows rows
    Mask &low_col_block_mask(const Shape &s, i64 block, i64 low_dim) {
        Mask &m = low_mask(3, s, block, low_dim);
        if (m.msg.empty()) {
            m.msg.assign((size_t)slots, cplx(0, 0));
            for (i64 i = 0; i < s.rows; i++)
                for (i64 k = 0; k < s.width; k += s.cols)
                    for (i64 j = block * low_dim; j < (1 + block) * low_dim; j++) m.msg[(size_t)(i * s.width + k + j)] = 1;
        }
        return m;
    }
    // getLowColBlock -- HEMMer.cpp:2292-2311
    CtT get_low_col_block(const CtT &t, i64 col_block, i64 low_dim) {
        return CtT{mult_msg(t.ct, low_col_block_mask(t.sh, col_block, low_dim)), t.sh};
    }
    // getLowRowBlock -- HEMMer.cpp:2313-2332
    CtT get_low_row_block(const CtT &t, i64 row_block, i64 low_dim) {
        Mask &m = low_mask(4, t.sh, row_block, low_dim);
        if (m.msg.empty()) {
            m.msg.assign((size_t)slots, cplx(0, 0));
            for (i64 i = row_block * low_dim; i < (1 + row_block) * low_dim; i++)
                for (i64 k = 0; k < t.sh.width; k += t.sh.cols)
                    for (i64 j = 0; j < t.sh.cols; j++) m.msg[(size_t)(i * t.sh.width + k + j)] = 1;
        }
        return CtT{mult_msg(t.ct, m), t.sh};
    }
};

} // namespace orc
