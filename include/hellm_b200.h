/* hellm_b200.h -- C entry points of libhellm_b200.so: the HELLM::HEMMer call surface on one B200.
 *
 * The reference exposes this surface as the C++ class HELLM::HEMMer
 * (ciphertext/include/HELLM/HEMMer.hpp:33-438) over HETensor values (HETensor.hpp:46-86); it
 * has no C ABI.  The same class, with the reference's method names, is in this repository's
 * csrc/hellm/HEMMer.hpp for C++ callers; the functions below are that class for callers that
 * bind through C.  Each one names the HEMMer method (header line) and the schedule it runs
 * (ciphertext/src/MatrixUtils.cpp or HEMMer.cpp lines).
 *
 * Conventions
 *   - a tile tensor travels as a ciphertext handle plus (rows, cols, block_width), the
 *     TileTensorShape of the reference (HETensor.hpp:16-44);
 *   - inputs are borrowed for the call, outputs are new caller-owned handles (hb_ct_free);
 *   - every function returns 0 or a negative HB_E_* code (hemmer_b200.h); the reference throws
 *     std::invalid_argument for shape and level violations (MatrixUtils.cpp:27,36,680,1113,1322),
 *     reported here as HB_E_ARG with the same message through hb_hemmer_last_error();
 *   - all ciphertext handles may hold a batch: every function applies the schedule to all batch
 *     members with one set of launches.
 */
#ifndef HELLM_B200_H
#define HELLM_B200_H

#include "hemmer_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct hb_hemmer hb_hemmer;

/* HEMMer::HEMMer over an existing context with keys (HEMMer.cpp:93-209); masks are cached per object */
int hb_hemmer_create(hb_ctx *ctx, hb_hemmer **out);
void hb_hemmer_destroy(hb_hemmer *h);
/* message of the last failure raised above the primitive layer (thread-local) */
const char *hb_hemmer_last_error(void);
/* 0: the reference's rotation sequence, each shifted copy rotated from the previous one (default);
 * 1: every shifted copy is one rotation of the transformed operand, sharing its decomposition;
 * 2: as 1, and each wrapped copy (two rotations, two masks, add, rescale) is one hb_assemble_masked; the operands
 *    of singleCCMatMul are levelled down before sigma / tau; inside the transforms every masked sum is rescaled
 *    once (hb_sum_mul_pt_rescale) and the giant-step rotations share one ModDown (hb_rotate_sum).
 * All give the same slots and different ciphertext bits; no counterpart in the reference. */
int hb_hemmer_set_schedule(hb_hemmer *h, int mode);

/* HEMMer::genHEMMer (HEMMer.hpp:38-44; HEMMer.cpp:93-112): creates the context on `device`, generates the keys and
 * builds the HEMMer in one call; hb_hemmer_destroy then releases the context too.  hb_hemmer_context gives the
 * primitive-layer handle of either kind of HEMMer. */
int hb_hemmer_gen(int device, const hb_params *prm, hb_hemmer **out);
hb_ctx *hb_hemmer_context(const hb_hemmer *h);
/* HEMMer::getRank / getMaxRank (HEMMer.hpp:56-57): this process's GPU among the GPUs of the job (set by the launcher) */
int hb_hemmer_set_rank(hb_hemmer *h, int rank, int max_rank);
int hb_hemmer_get_rank(const hb_hemmer *h);
int hb_hemmer_get_max_rank(const hb_hemmer *h);
/* HEMMer::save (HEMMer.hpp:61; HEMMer.cpp:225-230): secret key and switching keys to files under keys_path */
int hb_hemmer_save(hb_hemmer *h, const char *keys_path);

/* HEMMer::encode / encode2 / encodeDiagonalToRow4 (HEMMer.hpp:65-86; HEMMer.cpp:232-275, 353-416): row-major rows x cols
 * matrices of doubles instead of torch::Tensor; level 0 means the encryption level, as in the reference.  encode2 lays
 * [d1 | d2] side by side (block width 2 * cols); encodeDiagonalToRow4 packs 1/2 (w1 - i w3) | 1/2 (w2 - i w4) with
 * column j rolled up by j rows. */
int hb_hemmer_encode(hb_hemmer *h, const double *data, int rows, int cols, int level, hb_pt **out);
int hb_hemmer_encode2(hb_hemmer *h, const double *d1, const double *d2, int rows, int cols, int level, hb_pt **out);
int hb_hemmer_encode_diagonal_to_row4(hb_hemmer *h, const double *w1, const double *w2, const double *w3, const double *w4, int rows, int cols,
                                      int level, hb_pt **out);
/* HEMMer::encrypt / encrypt2 (HEMMer.hpp:93-94; HEMMer.cpp:579-594); `nonce` selects the random streams (the reference
 * draws unseeded randomness) */
int hb_hemmer_encrypt(hb_hemmer *h, const double *data, int rows, int cols, uint64_t nonce, hb_ct **out);
int hb_hemmer_encrypt2(hb_hemmer *h, const double *d1, const double *d2, int rows, int cols, uint64_t nonce, hb_ct **out);
/* HEMMer::decrypt / decrypt2 (HEMMer.hpp:98-100; HEMMer.cpp:603-638): rows * cols doubles, or [2][rows][cols] */
int hb_hemmer_decrypt(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, double *out);
int hb_hemmer_decrypt2(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, double *out);
/* HEMMer::addInplace / hadamardMultInplace (HEMMer.hpp:102-115; HEMMer.cpp:683-713), returning a new handle */
int hb_hemmer_add(hb_hemmer *h, const hb_ct *a, const hb_ct *b, hb_ct **out);
int hb_hemmer_hadamard_mult(hb_hemmer *h, const hb_ct *a, const hb_ct *b, hb_ct **out);
int hb_hemmer_hadamard_mult_pt(hb_hemmer *h, const hb_ct *a, const hb_pt *p, hb_ct **out);
/* HEMMer::oneMatRotSumInplace (HEMMer.hpp:168; HEMMer.cpp:882-919) on two-tile ciphertexts */
int hb_hemmer_one_mat_rot_sum(hb_hemmer *h, const hb_ct *a, const hb_ct *b, hb_ct **out_a, hb_ct **out_b);
/* HEMMer::tr_oneMatRotSumInplace (HEMMer.cpp:921-962, HEAD_DIM = tile side): after an optional level-down to target_level + 1,
 * a holds the sum of every tile row on the left half of the row, b on the right half. */
int hb_hemmer_tr_one_mat_rot_sum(hb_hemmer *h, const hb_ct *a, const hb_ct *b, int target_level, hb_ct **out_a, hb_ct **out_b);

/* HEMMer::maskFirstColInplace (which = 0), maskLeftHalfInplace (1), maskRightHalfInplace (2) -- HEMMer.cpp:1251-1269 */
int hb_hemmer_mask_inplace(hb_hemmer *h, const hb_ct *a, int which, int rows, int cols, int width, hb_ct **out);
/* HEMMer::squareSum (HEMMer.cpp:2499-2510): rescale(relinearize(sum_i tensor(v[i], v[i]))) */
int hb_hemmer_square_sum(hb_hemmer *h, const hb_ct *const *v, int count, int rows, int cols, int width, hb_ct **out);
/* HEMMer::reduceRowSumWithScaledMask (HEMMer.cpp:2512-2530) on one rank; `mask` is encoded at the ciphertext's level */
int hb_hemmer_reduce_row_sum_with_scaled_mask(hb_hemmer *h, const hb_ct *a, const hb_pt *mask, int rows, int cols, int width, hb_ct **out);
/* The score assembly of the Gaussian-kernel attention in the reference's layer, TransformerBlock::attention2_bert_loraOpti
 * (TransformerBlock.cpp:2420-2482, for one query / key pair, up to the bootstrap): heads separated by maskRightLeft,
 * squared norms by square + oneMatRotSumInplace (+ transposeInplace on the key side), the products by complexPacking* +
 * packedMatMul + repackCC; out_j = |q_r|^2 + |k_c|^2 - 2 q_r . k_c for head position j of both tiles, at target_level. */
int hb_hemmer_gaussian_kernel_scores(hb_hemmer *h, const hb_ct *query, const hb_ct *key, int rows, int cols, int width, int target_level,
                                     hb_ct **out0, hb_ct **out1);
/* The rank-2 LoRA branch of a projection in the reference's layer, TransformerBlock::attention2_bert_loraOpti
 * (TransformerBlock.cpp:2199-2365) without the bootstraps around it: X A by slot-wise products with the rank vectors
 * spread over the token rows and a rotate-and-add across each row, then (X A) B the same way.  cur0..2: the three
 * [X_2i | X_2i+1] activation pairs; lora_wa / lora_wb: two-tile ciphertexts whose row 2i+j holds rank vector j for
 * pair i.  out0..2: the three output pairs. */
int hb_hemmer_lora_opti_forward(hb_hemmer *h, const hb_ct *cur0, const hb_ct *cur1, const hb_ct *cur2, const hb_ct *lora_wa, const hb_ct *lora_wb,
                                hb_ct **out0, hb_ct **out1, hb_ct **out2);

/* HEMMer::transposeInplace (HEMMer.hpp:129; HEMMer.cpp:1166-1172; MatrixUtils.cpp:671-739) */
int hb_hemmer_transpose(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, int target_level, hb_ct **out);
/* MatrixTransformer::diagonalToColumn / diagonalToRow (MatrixUtils.cpp:776-848, 924-996) */
int hb_hemmer_sigma(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, hb_ct **out);
int hb_hemmer_tau(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, hb_ct **out);

/* HEMMer::singleCCMatMul (HEMMer.hpp:164-166; MatrixUtils.cpp:1307-1446) */
int hb_hemmer_matmul_cc(hb_hemmer *h, const hb_ct *a, int ra, int ca, int wa, const hb_ct *b, int rb, int cb, int wb,
                        int target_level, hb_ct **out);
/* the same product in two halves: the transforms (both results at target_level + 2), then the product loop.
 * Operands of different input levels can be transformed one by one and multiplied as one batch. */
int hb_hemmer_matmul_cc_prepare(hb_hemmer *h, const hb_ct *a, int ra, int ca, int wa, const hb_ct *b, int rb, int cb, int wb,
                                int target_level, hb_ct **sigma_a, hb_ct **tau_b);
int hb_hemmer_matmul_cc_core(hb_hemmer *h, const hb_ct *sigma_a, const hb_ct *tau_b, int rows, int inner, int cols, int width,
                             int target_level, hb_ct **out);
/* HEMMer::singleMatMul (HEMMer.hpp:160-162; MatrixUtils.cpp:1448-1570) */
int hb_hemmer_matmul_cp(hb_hemmer *h, const hb_ct *a, int ra, int ca, int wa, const hb_pt *b, int rb, int cb, int wb,
                        int target_level, hb_ct **out);
/* HEMMer::packedMatMul (HEMMer.cpp:833-838; MatrixUtils.cpp:1100-1216) */
int hb_hemmer_packed_matmul(hb_hemmer *h, const hb_ct *a, int ra, int ca, int wa, const hb_ct *b, int rb, int cb, int wb,
                            int target_level, hb_ct **out);

/* HEMMer::matMulPre (HEMMer.hpp:190-191; MatrixUtils.cpp:1572-1610): `out` is ONE handle whose batch holds the
 * shifted copies, copy k of input b at index k * batch(a) + b */
int hb_hemmer_matmul_pre(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, int target_level, hb_ct **out);
/* HEMMer::matMulReUse (HEMMer.hpp:192-194; MatrixUtils.cpp:1612-1639; HEaaN matmul, HomEvaluator.hpp:595-601) */
int hb_hemmer_matmul_reuse(hb_hemmer *h, const hb_ct *pre, const hb_pt *w, int rows, int cols, int width, hb_ct **out);
/* sum over `bcount` inputs b0.. of matMulReUse(copies of input b, pts[b - b0]) in one pass; `pre` holds the copies
 * of `btotal` inputs.  The sum the reference takes with addInplace over K tiles (bert-matmul.cpp:268-287). */
int hb_hemmer_matmul_reuse_groups(hb_hemmer *h, const hb_ct *pre, int btotal, int b0, const hb_pt *const *pts, int bcount,
                                  int width, hb_ct **out);
/* the same for `tiles` weights (pts[t * bcount + b]) that meet the same copies: out[t], t < tiles */
int hb_hemmer_matmul_reuse_groups_tiles(hb_hemmer *h, const hb_ct *pre, int btotal, int b0, const hb_pt *const *pts, int bcount, int tiles,
                                        int width, hb_ct **out);
/* HEMMer::matMulPreRev, matMulCCReUse (HEMMer.cpp:1114-1124; MatrixUtils.cpp:1641-1679) */
int hb_hemmer_matmul_pre_rev(hb_hemmer *h, const hb_ct *b, int rows, int cols, int width, int target_level, hb_ct **out);
int hb_hemmer_matmul_cc_reuse(hb_hemmer *h, const hb_ct *pre, const hb_ct *b, int rows, int cols, int width, hb_ct **out);
/* HEMMer::packedMatMulPre, PreRot, PreRev, CCReuse (HEMMer.cpp:840-864; MatrixUtils.cpp:1218-1305) */
int hb_hemmer_packed_matmul_pre(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, int target_level, hb_ct **out);
int hb_hemmer_packed_matmul_pre_rot(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, int target_level, hb_ct **out);
int hb_hemmer_packed_matmul_pre_rev(hb_hemmer *h, const hb_ct *b, int rows, int cols, int width, int target_level, hb_ct **out);
int hb_hemmer_packed_matmul_cc_reuse(hb_hemmer *h, const hb_ct *pre, const hb_ct *b, int rows, int cols, int width, hb_ct **out);

/* HEMMer::complexPackingInplace, complexPackingRowInplace, transposeComplexPackingInplace (HEMMer.cpp:764-817) */
int hb_hemmer_complex_packing(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, hb_ct **out);
int hb_hemmer_complex_packing_row(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, hb_ct **out);
int hb_hemmer_transpose_complex_packing(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, int target_level, hb_ct **out);
/* HEMMer::splitInTwo (HEMMer.cpp:819-831) */
int hb_hemmer_split_in_two(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, hb_ct **out1, hb_ct **out2);
/* HEMMer::repackCC (HEMMer.cpp:964-969), complexPacking(ct, ct) (:980-986), complexPackingRev (:988-994),
 * repack_notBTS (:1025-1053) */
int hb_hemmer_repack_cc(hb_hemmer *h, const hb_ct *a, hb_ct **out);
int hb_hemmer_complex_packing2(hb_hemmer *h, const hb_ct *a, const hb_ct *b, hb_ct **out);
int hb_hemmer_complex_packing_rev(hb_hemmer *h, const hb_ct *a, const hb_ct *b, hb_ct **out);
int hb_hemmer_repack_not_bts(hb_hemmer *h, const hb_ct *a, const hb_ct *b, hb_ct **out);
/* HEMMer::repack_loraOpti (HEMMer.cpp:1055-1091): repack_notBTS followed by the split of real and imaginary part
 * that the reference otherwise gets from bootstrapExtended */
int hb_hemmer_repack_lora_opti(hb_hemmer *h, const hb_ct *a, const hb_ct *b, hb_ct **out);

/* LoRA low-rank family.  `low_dim` is the width of the thin factor, ModelArgs::LOW_DIM in the reference
 * (ModelArgs.hpp:67, a compile-time 2 there); `in_*_block` / `block` is the index of the low_dim-wide column
 * (row) block the thin factor occupies inside its tile.
 * HEMMer::matMulHighLow / matMulLowHigh / matMulLowLow (HEMMer.hpp:326-334; MatrixUtils.cpp:1681-1996) */
int hb_hemmer_matmul_high_low(hb_hemmer *h, const hb_ct *a, int ra, int ca, int wa, const hb_ct *b, int rb, int cb, int wb,
                              int in_col_block, int target_level, int low_dim, hb_ct **out);
int hb_hemmer_matmul_low_high(hb_hemmer *h, const hb_ct *a, int ra, int ca, int wa, const hb_ct *b, int rb, int cb, int wb,
                              int in_row_block, int target_level, int low_dim, hb_ct **out);
int hb_hemmer_matmul_low_low(hb_hemmer *h, const hb_ct *a, int ra, int ca, int wa, const hb_ct *b, int rb, int cb, int wb,
                             int in_col_block, int in_row_block, int target_level, int low_dim, hb_ct **out);
/* HEMMer::repackToOneCol / MultiCol / OneRow / MultiRow (HEMMer.hpp:336-343; HEMMer.cpp:2131-2290): fold the
 * partial sums the products above leave spread over the blocks into block `block` */
int hb_hemmer_repack_to_one_col(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, int block, int low_dim, hb_ct **out);
int hb_hemmer_repack_to_multi_col(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, int block, int low_dim, hb_ct **out);
int hb_hemmer_repack_to_one_row(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, int block, int low_dim, hb_ct **out);
int hb_hemmer_repack_to_multi_row(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, int block, int low_dim, hb_ct **out);
/* HEMMer::getLowColBlock / getLowRowBlock (HEMMer.hpp:345-346; HEMMer.cpp:2292-2332): keep one block of every tile */
int hb_hemmer_low_col_block(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, int block, int low_dim, hb_ct **out);
int hb_hemmer_low_row_block(hb_hemmer *h, const hb_ct *a, int rows, int cols, int width, int block, int low_dim, hb_ct **out);

#ifdef __cplusplus
}
#endif
#endif /* HELLM_B200_H */
