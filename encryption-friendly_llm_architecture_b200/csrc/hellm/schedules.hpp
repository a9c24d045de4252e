// Matrix-multiplication schedules over encrypted tiles (the role of ciphertext/src/MatrixUtils.cpp).
#pragma once
#include "HEMMer.hpp"

namespace HELLM {
namespace sched {

// mask families, used as the first component of MaskCache::Key
enum MaskKind { kDiagonal = 0, kHorizontal, kVertical, kPackedHorizontal, kPackedVertical, kColWrap, kRowWrap, kHemmer };

struct Env { // what a schedule needs: evaluator, slot count, mask cache
    const Evaluator &ev;
    i64 slots;
    MaskCache &cache;
};

CtxtTensor transpose(Env &e, const CtxtTensor &op);
CtxtTensor diagonalToColumn(Env &e, const CtxtTensor &op);
CtxtTensor diagonalToRow(Env &e, const CtxtTensor &op);
CtxtTensor packedDiagonalToColumn(Env &e, const CtxtTensor &op);
CtxtTensor packedDiagonalToRow(Env &e, const CtxtTensor &op);

CtxtTensor multMatMatCC(Env &e, const CtxtTensor &a, const CtxtTensor &b, int target_level);
CtxtTensor multPackedMatMat(Env &e, const CtxtTensor &a, const CtxtTensor &b, int target_level);
CtxtTensor multPackedMatMatPre(Env &e, const CtxtTensor &a, int target_level);
Ciphertext multPackedMatMatPreRot(Env &e, const CtxtTensor &a, int target_level);
CtxtTensor multPackedMatMatPreRev(Env &e, const CtxtTensor &b, int target_level);
CtxtTensor multPackedMatMatCCReuse(Env &e, const Ciphertext &pre, const CtxtTensor &b);
Ciphertext multMatMatPre(Env &e, const CtxtTensor &a, int target_level);
CtxtTensor multMatMatReUse(Env &e, const Ciphertext &pre, const PtxtTensor &w);
CtxtTensor multMatMatPreRev(Env &e, const CtxtTensor &b, int target_level);
CtxtTensor multMatMatCCReUse(Env &e, const Ciphertext &pre, const CtxtTensor &b);

} // namespace sched
} // namespace HELLM
