// HELLM::HEMMer for B200 -- the call surface of ciphertext/include/HELLM/HEMMer.hpp
// (matmul entry points, transposes, packing helpers, encode / encrypt / decrypt) over the
// CUDA C ABI.  Matrices cross this interface as row-major double arrays instead of
// torch::Tensor, so the layer has no libtorch dependency.
#pragma once
#include "he_types.hpp"

#include <map>
#include <tuple>
#include <vector>

namespace HELLM {

// include/HELLM/HETensor.hpp:16-44
class TileTensorShape {
  public:
    TileTensorShape() = default;
    TileTensorShape(i64 rows, i64 cols, i64 block_width) : rows_(rows), cols_(cols), width_(block_width) {}
    TileTensorShape(i64 rows, i64 cols) : rows_(rows), cols_(cols), width_(1) { while (width_ < cols) width_ <<= 1; }
    i64 getNumRows() const { return rows_; }
    i64 getNumCols() const { return cols_; }
    i64 getBlockWidth() const { return width_; }
    void setShape(i64 r, i64 c) { rows_ = r; cols_ = c; }
    void setBlockWidth(i64 w) { width_ = w; }
    bool operator<(const TileTensorShape &o) const { return std::tie(rows_, cols_, width_) < std::tie(o.rows_, o.cols_, o.width_); }
  private:
    i64 rows_ = 0, cols_ = 0, width_ = 0;
};

// include/HELLM/HETensor.hpp:46-86
template <class T> class HETensor {
  public:
    HETensor() = default;
    HETensor(TileTensorShape s, T data) : shape_(s), data_(std::move(data)) {}
    HETensor(i64 h, i64 w, T data) : shape_(h, w), data_(std::move(data)) {}
    HETensor(i64 h, i64 w, T data, i64 block_width) : shape_(h, w, block_width), data_(std::move(data)) {}
    i64 getHeight() const { return shape_.getNumRows(); }
    i64 getWidth() const { return shape_.getNumCols(); }
    i64 getBlockWidth() const { return shape_.getBlockWidth(); }
    int getLevel() const { return data_.getLevel(); }
    void setShape(i64 h, i64 w) { shape_.setShape(h, w); }
    TileTensorShape getShape() const { return shape_; }
    T &get() { return data_; }
    const T &get() const { return data_; }
  private:
    TileTensorShape shape_;
    T data_;
};
using CtxtTensor = HETensor<Ciphertext>;
using PtxtTensor = HETensor<Plaintext>;

// Masks of the linear transforms: cleartext slot vectors, encoded once per level and kept on the
// device.  (The reference keeps Messages and lets HEaaN re-encode them inside every multiplication,
// MatrixUtils.cpp:584-669; encoding is deterministic, so the ciphertexts are the same.)
class MaskCache {
  public:
    using Key = std::tuple<int, TileTensorShape, i64, int>; // kind, shape, index, level
    const Plaintext *find(const Key &k) const { auto it = enc_.find(k); return it == enc_.end() ? nullptr : &it->second; }
    const Plaintext &put(const Key &k, Plaintext p) { return enc_.emplace(k, std::move(p)).first->second; }
    // rotation keys that carry a wrap mask (schedule 2), per (kind, shape, shift index, level)
    const MaskedKey *findKey(const Key &k) const { auto it = keys_.find(k); return it == keys_.end() ? nullptr : &it->second; }
    const MaskedKey &putKey(const Key &k, MaskedKey m) { return keys_.emplace(k, std::move(m)).first->second; }
    void clear() { enc_.clear(); keys_.clear(); }
  private:
    std::map<Key, Plaintext> enc_;
    std::map<Key, MaskedKey> keys_;
};

class HEMMer {
  public:
    // Wraps an existing context (keys must have been generated with hb_keygen).
    explicit HEMMer(hb_ctx *ctx);
    // HEMMer::genHEMMer (HEMMer.cpp:93-112): creates the context on `device_id`, generates keys; owns the context.
    static HEMMer *genHEMMer(int device_id, const hb_params &prm);
    ~HEMMer();

    const Evaluator &eval() const { return eval_; }
    i64 slots() const { return slots_; }
    i64 tile() const { return tile_; }
    int encryptionLevel() const { return max_level_; }

    // encode / encrypt / decrypt -- HEMMer.cpp:232-275, 353-416, 579-638
    Message message2(const double *d1, const double *d2, i64 h, i64 w) const;
    Message msgDiagonalToRow4(const double *w1, const double *w2, const double *w3, const double *w4, i64 h, i64 w) const;
    PtxtTensor encode(const double *data, i64 h, i64 w, int level = 0) const;
    PtxtTensor encode2(const double *d1, const double *d2, i64 h, i64 w, int level = 0) const;
    PtxtTensor encodeDiagonalToRow4(const double *w1, const double *w2, const double *w3, const double *w4, i64 h, i64 w, int level = 0) const;
    CtxtTensor encrypt(const double *data, i64 h, i64 w, u64 nonce) const;
    CtxtTensor encrypt2(const double *d1, const double *d2, i64 h, i64 w, u64 nonce) const;
    void decrypt(const CtxtTensor &t, double *out) const;  // h*w doubles
    void decrypt2(const CtxtTensor &t, double *out) const; // [2][h][w]

    void addInplace(CtxtTensor &a, const CtxtTensor &b) const;
    // HEMMer::hadamardMultInplace (HEMMer.hpp:107-115; HEMMer.cpp:702-713): slot-wise product, ciphertext or plaintext operand
    void hadamardMultInplace(CtxtTensor &a, const CtxtTensor &b) const;
    void hadamardMultInplace(CtxtTensor &a, const PtxtTensor &b) const;
    // HEMMer::oneMatRotSumInplace (HEMMer.cpp:882-919): row sums of the left half of a's tiles and of the right half of
    // b's tiles, spread over every column -- the norm terms of the Gaussian-kernel attention scores
    void oneMatRotSumInplace(CtxtTensor &a, CtxtTensor &b);
    // HEMMer::tr_oneMatRotSumInplace (HEMMer.cpp:921-962): row sums over the whole tile side, returned on half of it
    void trOneMatRotSumInplace(CtxtTensor &a, CtxtTensor &b, int target_level = 0);
    // HEMMer::maskFirstColInplace / maskLeftHalfInplace / maskRightHalfInplace (HEMMer.cpp:1251-1269)
    void maskFirstColInplace(CtxtTensor &t);
    void maskLeftHalfInplace(CtxtTensor &t);
    void maskRightHalfInplace(CtxtTensor &t);
    // HEMMer::squareSum (HEMMer.cpp:2499-2510)
    void squareSum(const std::vector<CtxtTensor> &v, CtxtTensor &out);
    // HEMMer::reduceRowSumWithScaledMask (HEMMer.cpp:2512-2530), single rank; the mask comes encoded at the ciphertext's level
    void reduceRowSumWithScaledMask(CtxtTensor &t, const PtxtTensor &mask);
    // The rank-2 LoRA branch of a projection as the reference's layer runs it (TransformerBlock::attention2_bert_loraOpti,
    // TransformerBlock.cpp:2199-2365, without the bootstraps around it): the two rank vectors are picked row by row
    // out of the factor ciphertexts, spread over all token rows by rotations, multiplied slot-wise with the three
    // activation pairs and summed across the row (X A), then spread across the row again and multiplied with the
    // rows of the second factor ((X A) B).  cur: three [X_2i | X_2i+1] pairs; wa / wb: row 2i+j of the two-tile
    // ciphertext holds rank vector j for pair i.  Returns the three output pairs.
    std::vector<CtxtTensor> loraOptiForward(const std::vector<CtxtTensor> &cur, const CtxtTensor &lora_wa, const CtxtTensor &lora_wb);
    // The score assembly of the Gaussian-kernel attention in the reference's layer (TransformerBlock::attention2_bert_loraOpti,
    // TransformerBlock.cpp:2420-2482, up to the bootstrap): a two-tile ciphertext holds two heads per tile (columns 0..d/2-1
    // and d/2..d-1).  maskRightLeft separates the heads, square + oneMatRotSumInplace give |q_r|^2 spread over the rows
    // and (after a transpose) |k_c|^2 spread over the columns, complexPacking* + packedMatMul + repackCC give q_r . k_c,
    // and the result is |q_r|^2 + |k_c|^2 - 2 q_r . k_c.  Returns one ciphertext per head position, at target_level.
    std::vector<CtxtTensor> gaussianKernelScores(const CtxtTensor &query, const CtxtTensor &key, int target_level = 4);
    // HEMMer::maskRightLeft (HEMMer.cpp, masks :2366-2376): the first / second head of every tile
    void maskRightLeft(const CtxtTensor &t, CtxtTensor &left, CtxtTensor &right);
    // HEMMer::maskFirstRowInplace / maskFirstColOnlyInplace (HEMMer.cpp:1255-1261)
    void maskFirstRowInplace(CtxtTensor &t);
    void maskFirstColOnlyInplace(CtxtTensor &t);
    // HEMMer::getRank / getMaxRank (HEMMer.hpp:56-57): this process's GPU among the GPUs of the job
    int getRank() const { return rank_; }
    int getMaxRank() const { return max_rank_; }
    void setRank(int rank, int max_rank) { rank_ = rank; max_rank_ = max_rank; }
    // HEMMer::save (HEMMer.cpp:225-230): secret key and switching keys to `keys_path` (hb_keys_save)
    void save(const std::string &keys_path) const;
    hb_ctx *context() const { return ctx_; }
    // matmul family -- HEMMer.cpp:833-880, 1102-1124
    CtxtTensor singleCCMatMul(const CtxtTensor &a, const CtxtTensor &b, int target_level = 4);
    CtxtTensor singleMatMul(const CtxtTensor &a, const PtxtTensor &b, int target_level = 4);
    // singleCCMatMul in two halves (transforms, then the product loop), for batching operands of different levels
    void ccMatMulPrepare(const CtxtTensor &a, const CtxtTensor &b, int target_level, Ciphertext &sigma_a, Ciphertext &tau_b);
    CtxtTensor ccMatMulCore(Ciphertext sigma_a, Ciphertext tau_b, i64 rows, i64 inner, i64 cols, i64 width, int target_level);
    CtxtTensor packedMatMul(const CtxtTensor &a, const CtxtTensor &b, int target_level = 4);
    CtxtTensor packedMatMulPre(const CtxtTensor &a, int target_level = 4);
    Ciphertext packedMatMulPreRot(const CtxtTensor &a, int target_level = 4);
    CtxtTensor packedMatMulPreRev(const CtxtTensor &b, int target_level = 4);
    CtxtTensor packedMatMulCCReuse(const Ciphertext &pre, const CtxtTensor &b, int target_level = 4);
    Ciphertext matMulPre(const CtxtTensor &a, int target_level = 4);
    CtxtTensor matMulReUse(const Ciphertext &pre, const PtxtTensor &w, int target_level = 4);
    CtxtTensor matMulPreRev(const CtxtTensor &b, int target_level = 4);
    CtxtTensor matMulCCReUse(const Ciphertext &pre, const CtxtTensor &b, int target_level = 4);
    // transposes and packing -- HEMMer.cpp:764-831, 964-1053, 1166-1172
    void transposeInplace(CtxtTensor &t, int target_level = 0);
    void complexPackingInplace(CtxtTensor &t);
    void transposeComplexPackingInplace(CtxtTensor &t, int target_level = 0);
    void complexPackingRowInplace(CtxtTensor &t);
    void splitInTwo(const CtxtTensor &t, CtxtTensor &t1, CtxtTensor &t2);
    CtxtTensor repackCC(const CtxtTensor &t) const;
    CtxtTensor complexPacking(const CtxtTensor &a, const CtxtTensor &b) const;
    CtxtTensor complexPackingRev(const CtxtTensor &a, const CtxtTensor &b) const;
    CtxtTensor repack_notBTS(const CtxtTensor &a, const CtxtTensor &b);
    CtxtTensor repack_loraOpti(const CtxtTensor &a, const CtxtTensor &b);
    // LoRA low-rank products and their repacking -- HEMMer.cpp:2108-2332.  The thin factor has lowDim() columns or
    // rows (ModelArgs::LOW_DIM, ModelArgs.hpp:67) and sits in block `in_*_block` of its tile.
    CtxtTensor matMulHighLow(const CtxtTensor &a, const CtxtTensor &b, u64 in_col_block, int target_level = 4);
    CtxtTensor matMulLowHigh(const CtxtTensor &a, const CtxtTensor &b, u64 in_row_block, int target_level = 4);
    CtxtTensor matMulLowLow(const CtxtTensor &a, const CtxtTensor &b, u64 in_col_block, u64 in_row_block, int target_level = 4);
    CtxtTensor repackToOneCol(const CtxtTensor &t, u64 out_col_block);
    CtxtTensor repackToMultiCol(const CtxtTensor &t, u64 out_col_block);
    CtxtTensor repackToOneRow(const CtxtTensor &t, u64 out_row_block);
    CtxtTensor repackToMultiRow(const CtxtTensor &t, u64 out_row_block);
    CtxtTensor getLowColBlock(const CtxtTensor &t, u64 col_block);
    CtxtTensor getLowRowBlock(const CtxtTensor &t, u64 row_block);
    void setLowDim(i64 low_dim) { low_dim_ = low_dim; }
    i64 lowDim() const { return low_dim_; }
    // the two linear transforms on their own (MatrixTransformer::diagonalToColumn / diagonalToRow)
    CtxtTensor diagonalToColumn(const CtxtTensor &t);
    CtxtTensor diagonalToRow(const CtxtTensor &t);

    MaskCache &masks() { return masks_; }
    // 0: the reference's rotation sequence; 1: direct (hoisted) rotations -- see sched::ScheduleMode
    void setSchedule(int mode) { schedule_ = mode; }
    int schedule() const { return schedule_; }

  private:
    hb_ctx *ctx_;
    bool owns_ctx_ = false;
    Evaluator eval_;
    i64 slots_ = 0, tile_ = 0;
    int max_level_ = 0;
    int schedule_ = 0;
    i64 low_dim_ = 2;
    int rank_ = 0, max_rank_ = 1;
    MaskCache masks_;
};

} // namespace HELLM
