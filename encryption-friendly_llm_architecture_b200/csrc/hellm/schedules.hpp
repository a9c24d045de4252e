// Matrix-multiplication schedules over encrypted tiles (the role of ciphertext/src/MatrixUtils.cpp).
#pragma once
#include "HEMMer.hpp"

namespace HELLM {
namespace sched {

// mask families, used as the first component of MaskCache::Key
enum MaskKind { kDiagonal = 0, kHorizontal, kVertical, kPackedHorizontal, kPackedVertical, kColWrap, kRowWrap, kHemmer, kLowRank, kColWrapKey, kRowWrapKey };

// Schedule variants.  kFaithful keeps the reference's sequence of rotations (each shifted copy is the previous one
// rotated once more).  kDirect takes every shifted copy straight from the transformed operand, rot(x, k) instead of
// rot(rot(...), 1): the same slots, fewer chained key switches (less noise), and all rotations of one ciphertext
// share the step-independent half of the key switch (hoisting).  The two variants give different ciphertext bits;
// the CPU oracle implements both so that each can be checked bit for bit.
// kLazy is kDirect with the masked pair of rotations that makes a wrapped copy done as one operation
// (Evaluator::assembleRotations): the two key switches stay in the extended basis, the masks are applied there, and
// one division by P * q_level replaces two ModDowns and a rescale -- in the product loop and in multMatMatPre.
// multMatMat also brings its operands down to target + 3 before sigma / tau (the reference transforms at the
// operands' level and levels down afterwards): the same slots from transforms on far fewer limbs.  The masked sums of
// the baby-step / giant-step transforms are rescaled once per sum (the reference rescales every term), and their
// giant-step rotations are summed in the extended basis before ONE ModDown (Evaluator::rotateSum).
enum ScheduleMode { kFaithful = 0, kDirect = 1, kLazy = 2 };

struct Env { // what a schedule needs: evaluator, slot count, mask cache, variant
    const Evaluator &ev;
    i64 slots;
    MaskCache &cache;
    int mode = kFaithful;
};

CtxtTensor transpose(Env &e, const CtxtTensor &op);
CtxtTensor diagonalToColumn(Env &e, const CtxtTensor &op);
CtxtTensor diagonalToRow(Env &e, const CtxtTensor &op);
CtxtTensor packedDiagonalToColumn(Env &e, const CtxtTensor &op);
CtxtTensor packedDiagonalToRow(Env &e, const CtxtTensor &op);

CtxtTensor multMatMatCC(Env &e, const CtxtTensor &a, const CtxtTensor &b, int target_level);
void ccmmPrepare(Env &e, const CtxtTensor &a, const CtxtTensor &b, int target_level, Ciphertext &sigma_a, Ciphertext &tau_b);
CtxtTensor ccmmCore(Env &e, Ciphertext sigma_a, Ciphertext tau_b, i64 rows, i64 inner, i64 cols, i64 width, int target_level);
CtxtTensor multMatMatCP(Env &e, const CtxtTensor &a, const PtxtTensor &b, int target_level);
CtxtTensor multPackedMatMat(Env &e, const CtxtTensor &a, const CtxtTensor &b, int target_level);
CtxtTensor multPackedMatMatPre(Env &e, const CtxtTensor &a, int target_level);
Ciphertext multPackedMatMatPreRot(Env &e, const CtxtTensor &a, int target_level);
CtxtTensor multPackedMatMatPreRev(Env &e, const CtxtTensor &b, int target_level);
CtxtTensor multPackedMatMatCCReuse(Env &e, const Ciphertext &pre, const CtxtTensor &b);
Ciphertext multMatMatPre(Env &e, const CtxtTensor &a, int target_level);
CtxtTensor multMatMatReUse(Env &e, const Ciphertext &pre, const PtxtTensor &w);
CtxtTensor multMatMatPreRev(Env &e, const CtxtTensor &b, int target_level);
CtxtTensor multMatMatCCReUse(Env &e, const Ciphertext &pre, const CtxtTensor &b);
// LoRA low-rank products (MatrixUtils.cpp:1681-1996); low_dim stands for ModelArgs::LOW_DIM
CtxtTensor multMatMatHighLow(Env &e, const CtxtTensor &a, const CtxtTensor &b, i64 in_col_block, int target_level, i64 low_dim);
CtxtTensor multMatMatLowHigh(Env &e, const CtxtTensor &a, const CtxtTensor &b, i64 in_row_block, int target_level, i64 low_dim);
CtxtTensor multMatMatLowLow(Env &e, const CtxtTensor &a, const CtxtTensor &b, i64 in_col_block, i64 in_row_block, int target_level, i64 low_dim);

} // namespace sched
} // namespace HELLM
