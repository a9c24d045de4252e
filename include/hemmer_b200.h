/* hemmer_b200.h -- C ABI of libhemmer_b200.so: RNS-CKKS primitives on one B200.
 *
 * The reference reaches its GPU arithmetic through the C++ classes of the closed HEaaN
 * library (headers under ciphertext/external/include/HEaaN/).  There is no C ABI in the
 * reference; each entry point below names the HEaaN call (header:line) whose role it
 * takes.  The C++ HELLM::HEMMer layer of this repository calls only these functions.
 *
 * Conventions
 *   - every function returns 0 on success or a negative HB_E_* code; hb_last_error()
 *     gives a message for the last failure on that context;
 *   - handles are caller-owned and released with hb_ct_free / hb_pt_free / hb_ctx_destroy;
 *   - a ciphertext handle holds a BATCH of `batch` independent ciphertexts of equal level,
 *     device layout [batch][poly][limb][N] of uint64 residues in NTT form, fully reduced;
 *   - a context is used from one host thread at a time; all work runs on one CUDA stream;
 *   - nothing here falls back to the CPU: without a CUDA device hb_ctx_create fails.
 */
#ifndef HEMMER_B200_H
#define HEMMER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct hb_ctx hb_ctx;
typedef struct hb_ct hb_ct;
typedef struct hb_pt hb_pt;
typedef struct hb_digits hb_digits;
typedef struct hb_mkey hb_mkey;

enum {
    HB_OK = 0,
    HB_E_ARG = -1,      /* bad argument (std::invalid_argument in the reference, MatrixUtils.cpp:27,36,680) */
    HB_E_LEVEL = -2,    /* level too low / mismatch (MatrixUtils.cpp:1320-1324) */
    HB_E_SHAPE = -3,    /* batch / poly-count / scale mismatch */
    HB_E_NOKEY = -4,    /* rotation key missing (HEaaN RuntimeException) */
    HB_E_CUDA = -5,     /* CUDA runtime error */
    HB_E_OOM = -6,      /* device allocation failed */
    HB_E_NCCL = -7,     /* collective failed */
    HB_E_TIMEOUT = -8,  /* a bounded device-side wait gave up */
    HB_E_LIMIT = -9     /* size beyond a fixed capacity */
};

/* Parameters; HEaaN fixes them through ParameterPreset::FGb (ParameterPreset.hpp:34, HEMMer.hpp:36). */
typedef struct hb_params {
    int32_t log_n;          /* ring degree N = 2^log_n */
    int32_t max_level;      /* L: moduli q_0..q_L */
    int32_t dnum;           /* gadget rank (Context.hpp:43-87) */
    int32_t num_special;    /* K special primes */
    int32_t q0_bits, q_bits, p_bits;
    int32_t hamming_weight;
    double sigma;
    uint64_t seed[4];       /* ChaCha20 key for every random stream (Randomseeds.hpp:26) */
} hb_params;

/* makeContext(preset, {device}) -- Context.hpp:88-92 */
int hb_ctx_create(const hb_params *prm, int device, hb_ctx **out);
void hb_ctx_destroy(hb_ctx *ctx);
const char *hb_last_error(const hb_ctx *ctx);
/* getPrimeList / scale factors -- Context.hpp:203-206.  primes[L+1+K], scales[L+1]. */
int hb_ctx_info(const hb_ctx *ctx, uint64_t *primes, double *scales);
/* getDegree / getEncryptionLevel -- Context.hpp:169-194 */
int hb_ctx_dims(const hb_ctx *ctx, int *log_n, int *max_level, int *num_special);
/* CudaTools::cudaDeviceSynchronize -- HEaaN/device/CudaTools.hpp:24 */
int hb_sync(hb_ctx *ctx);
/* bytes currently held by the context's device pool (cudaMemGetInfo print in bert-matmul.cpp:240-243) */
int hb_mem_info(const hb_ctx *ctx, uint64_t *pool_bytes, uint64_t *in_use_bytes);
/* Launches one warp that waits, with a limit of 64 polls, on a barrier nothing completes.  The wait gives up, the kernel
 * returns, and the next hb_sync reports HB_E_TIMEOUT once; the context stays usable.  Exercises the path every bounded
 * device-side wait of the library takes when a copy does not land. */
int hb_selftest_bounded_wait(hb_ctx *ctx);
/* hands the pool's idle device buffers back to the driver (the buffers of live handles stay); refused while a graph records */
int hb_release_cached(hb_ctx *ctx);
/* the CUDA stream all kernels of this context run on (as a void* cudaStream_t) */
void *hb_stream(const hb_ctx *ctx);
/* number of kernels this context has launched since creation */
uint64_t hb_launch_count(const hb_ctx *ctx);
/* Compulsory HBM traffic, in bytes, of the primitives this context has run since creation: every input of a primitive
 * (rotation, rescale, tensor, relinearise, plaintext product, fused accumulate ...) read once, every output written
 * once, a switching key or plaintext once per batch; the transforms and temporaries inside a primitive do not count.
 * Divided by the HBM bandwidth it is the time a call sequence cannot go below ("schedule roofline"). */
uint64_t hb_algorithmic_bytes(const hb_ctx *ctx);

/* KeyGenerator::genCommonKeys -- KeyGenerator.hpp:160-165: secret, multiplication and conjugation keys */
int hb_keygen(hb_ctx *ctx);
/* KeyGenerator::genRotKeyBundle -- KeyGenerator.hpp:89.  One direct key per left-rotation step. */
int hb_gen_rot_keys(hb_ctx *ctx, const int64_t *left_steps, int n);
/* copy a switching key to the host: galois = 0 selects the multiplication key.
 * Layout [digit][2][L+1+K][N]; *digits receives the digit count when host == NULL. */
int hb_evk_export(hb_ctx *ctx, uint64_t galois, uint64_t *host, int *digits);
uint64_t hb_galois_for_rotation(const hb_ctx *ctx, int64_t left_steps);

/* EnDecoder::encode / decode -- EnDecoder.hpp:51,66.  im may be NULL (real message). */
int hb_encode(hb_ctx *ctx, const double *re, const double *im, size_t n_slots, int level, hb_pt **out);
int hb_decode(hb_ctx *ctx, const hb_pt *pt, double *re, double *im);
/* hb_encode with K further limbs modulo the special primes after the level + 1 usual ones: the plaintext operand of
 * hb_assemble_rot.  Usable wherever a plaintext of that level is.  No counterpart in the reference. */
int hb_encode_ext(hb_ctx *ctx, const double *re, const double *im, size_t n_slots, int level, hb_pt **out);
/* Encryptor::encrypt(ptxt, sk, ctxt) -- Encryptor.hpp:84; `nonce` selects the random streams */
int hb_encrypt(hb_ctx *ctx, const hb_pt *pt, uint64_t nonce, hb_ct **out);
/* encode + encrypt `count` messages (message i at re + i * n_slots, im likewise or NULL) into ONE handle of batch
 * `count`: the inverse embeddings and error polynomials are made on the host cores in parallel, uploaded in one
 * copy, and the device part runs over the whole batch.  Member i is bit for bit hb_encrypt(hb_encode(message i,
 * level), nonces[i]). */
int hb_encrypt_many(hb_ctx *ctx, const double *re, const double *im, size_t n_slots, int count, int level, const uint64_t *nonces,
                    hb_ct **out);
/* Decryptor::decrypt -- Decryptor.hpp:36; decrypts entry `index` of the batch */
int hb_decrypt(hb_ctx *ctx, const hb_ct *ct, int index, double *re, double *im);
/* the same for `count` ciphertexts at once (member index[i] of batch handle cts[i]; index may be NULL for all zero):
 * one device pass and one copy for all, the CRT lift and the inverse embedding spread over the host cores.
 * re / im receive count * slots doubles; each member's values are exactly those hb_decrypt gives. */
int hb_decrypt_many(hb_ctx *ctx, const hb_ct *const *cts, const int *index, int count, double *re, double *im);

/* Ciphertext construction / metadata / raw residues -- Ciphertext.hpp:83-131 */
int hb_ct_create(hb_ctx *ctx, int level, int n_poly, int batch, int scale_pow, hb_ct **out);
int hb_ct_clone(hb_ctx *ctx, const hb_ct *src, hb_ct **out);
int hb_ct_zero(hb_ctx *ctx, hb_ct *ct); /* all residues 0: an encryption of zero with zero noise */
void hb_ct_free(hb_ct *ct);
void hb_pt_free(hb_pt *pt);
int hb_ct_meta(const hb_ct *ct, int *level, int *n_poly, int *batch, int *scale_pow);
int hb_pt_meta(const hb_pt *pt, int *level, int *scale_pow);
int hb_ct_import(hb_ctx *ctx, hb_ct *ct, const uint64_t *host);
int hb_ct_export(hb_ctx *ctx, const hb_ct *ct, uint64_t *host);
int hb_pt_export(hb_ctx *ctx, const hb_pt *pt, uint64_t *host);
void *hb_ct_device_ptr(const hb_ct *ct);
/* Files.  HEaaN's binary format is not published, so these calls write and read this library's own container:
 * a 96-byte header (magic, kind, ring degree, level, polynomial count, batch, scale power, a hash of the primes),
 * the plain residues in device layout, and a checksum.  A file is accepted only under the parameters it was
 * written with.  hb_ct_save / hb_ct_load stand for Ciphertext::save / load (Ciphertext.hpp:89-98; the reference keeps
 * forward-pass activations for the backward pass this way, HEMMer.cpp:1403-1405, TransformerBlock.cpp:11059-11079);
 * hb_pt_save / hb_pt_load for Plaintext::save / load (encoded weights, HEMMer::encodeWeight); hb_keys_save for
 * HEMMer::save (HEMMer.cpp:225-230): SecretKey.bin, MultKey.bin and one GaloisKey_<galois>.bin per generated key under
 * an existing directory; hb_keys_load reads them back (the Galois keys named in `galois`). */
int hb_ct_save(hb_ctx *ctx, const hb_ct *ct, const char *path);
int hb_ct_load(hb_ctx *ctx, const char *path, hb_ct **out);
int hb_pt_save(hb_ctx *ctx, const hb_pt *pt, const char *path);
int hb_pt_load(hb_ctx *ctx, const char *path, hb_pt **out);
int hb_keys_save(hb_ctx *ctx, const char *dir);
int hb_keys_load(hb_ctx *ctx, const char *dir, const uint64_t *galois, int count);
/* copies all of src's entries to positions index*src_batch .. of dst */
int hb_batch_set(hb_ctx *ctx, hb_ct *dst, int index, const hb_ct *src);
int hb_batch_get(hb_ctx *ctx, const hb_ct *src, int index, hb_ct **out);
/* join batches end to end / copy out a run of entries (device-to-device copies) */
int hb_batch_concat(hb_ctx *ctx, const hb_ct *const *parts, int n, hb_ct **out);
int hb_batch_slice(hb_ctx *ctx, const hb_ct *src, int start, int count, hb_ct **out);

/* HomEvaluator primitives; `out` receives a new handle unless stated otherwise. */
int hb_add(hb_ctx *ctx, const hb_ct *a, const hb_ct *b, hb_ct **out);           /* HomEvaluator.hpp:143-146 */
int hb_sub(hb_ctx *ctx, const hb_ct *a, const hb_ct *b, hb_ct **out);           /* :222-225 */
int hb_negate(hb_ctx *ctx, const hb_ct *a, hb_ct **out);                        /* :66-68 */
int hb_mult_imag(hb_ctx *ctx, const hb_ct *a, hb_ct **out);                     /* multImagUnit :329-331 */
int hb_mult_int(hb_ctx *ctx, const hb_ct *a, int64_t k, hb_ct **out);           /* multInteger :346-348 */
int hb_mul_pt(hb_ctx *ctx, const hb_ct *a, const hb_pt *p, hb_ct **out);        /* mult(ct,ptxt) :299-301 */
int hb_mul_pt_norescale(hb_ctx *ctx, const hb_ct *a, const hb_pt *p, hb_ct **out); /* multWithoutRescale :490-493 */
int hb_rescale(hb_ctx *ctx, const hb_ct *a, hb_ct **out);                       /* rescale :539-540 */
int hb_level_down(hb_ctx *ctx, const hb_ct *a, int target, hb_ct **out);        /* levelDown :574-576 */
/* Rescale without any allocation (no counterpart in the reference).  For callers that may not obtain
 * device memory while they run -- a service whose device budget was handed out completely at start-up, or
 * a host that shares the GPU with an allocator it must not perturb.  Same result as hb_rescale, written
 * into the caller's `out` (created beforehand at level-1 with the same poly count and batch).  The
 * temporaries live in a 13 MiB buffer built into the library image, enough for one 2-poly ciphertext at
 * level 12 with N = 2^16 (poly_count * batch * level * N * 8 + poly_count * batch * N * 8 bytes are
 * needed); larger requests return HB_E_LIMIT.  The first call on a device looks the buffer's address up
 * and should therefore be made before any stream capture begins.  All calls share the buffer: nothing in
 * it has to start at zero (every word is written before it is read), but two calls that overlap on the
 * GPU -- different contexts or streams -- would corrupt each other, so issue them one after another. */
int hb_rescale_noalloc(hb_ctx *ctx, const hb_ct *a, hb_ct *out);
int hb_tensor(hb_ctx *ctx, const hb_ct *a, const hb_ct *b, hb_ct **out);        /* tensor :518 */
int hb_relin(hb_ctx *ctx, const hb_ct *a, hb_ct **out);                         /* relinearize :524 */
int hb_mul(hb_ctx *ctx, const hb_ct *a, const hb_ct *b, hb_ct **out);           /* mult(ct,ct) :311-312 */
int hb_square(hb_ctx *ctx, const hb_ct *a, hb_ct **out);                        /* square :363 */
int hb_mul_const(hb_ctx *ctx, const hb_ct *a, double re, double im, hb_ct **out); /* mult(ct, Complex / Real) :275-278 */
int hb_rotate(hb_ctx *ctx, const hb_ct *a, int64_t left_steps, hb_ct **out);    /* leftRotate :383 / rightRotate :403 */
int hb_conjugate(hb_ctx *ctx, const hb_ct *a, hb_ct **out);                     /* conjugate :465 */
/* Hoisted rotations: hb_decompose does the part of leftRotate that does not depend on the step (inverse NTT,
 * lift of every key-switch digit, forward NTT); hb_rotate_hoisted finishes one rotation from it.  The result is bit
 * for bit hb_rotate(a, left_steps): rotation is defined as decompose-then-permute.  (HEaaN exposes no such split;
 * the reference's loops call leftRotate once per step, MatrixUtils.cpp:1416-1420.) */
int hb_decompose(hb_ctx *ctx, const hb_ct *a, hb_digits **out);
int hb_rotate_hoisted(hb_ctx *ctx, const hb_ct *a, const hb_digits *digits, int64_t left_steps, hb_ct **out);
void hb_digits_free(hb_digits *digits);
/* out = sum_t rot(xs[t], left_steps[t]) for ciphertexts of equal level (at most 16 rotated and 16 unrotated terms): the key-switch inner products of
 * all terms are added up in the extended basis and ONE ModDown serves the sum (a step of 0 adds its operand as it is).
 * The giant-step half of a baby-step / giant-step transform in schedule 2.  Same slots as the sum of hb_rotate
 * results, different bits (one rounding instead of one per term); the oracle's Evaluator::rotate_sum is the same
 * arithmetic.  No counterpart in HEaaN. */
int hb_rotate_sum(hb_ctx *ctx, const hb_ct *const *xs, const int64_t *left_steps, int count, hb_ct **out);
/* The same when the terms are the member groups of ONE ciphertext (group t = members t * batch / groups onwards): the
 * digits of all groups are lifted by one batched call.  out has batch / groups members. */
int hb_rotate_sum_grouped(hb_ctx *ctx, const hb_ct *x, const int64_t *left_steps, int groups, hb_ct **out);
/* The masked pair of rotations that makes one wrapped copy in the shift loops (MatrixUtils.cpp:1416-1427:
 * two leftRotate, two multWithoutRescale, add, rescale) as one operation:
 *     out = p1 (.) rot(a, s1) + p2 (.) rot(a, s2),   at level(a) - 1.
 * Both key-switch inner products stay in the extended basis Q_level u P, are multiplied there by the extended
 * plaintexts (hb_encode_ext) and summed, and the sum is divided once by P * q_level -- instead of a ModDown per
 * rotation and a rescale of the sum.  Same slots as the unfused sequence, different ciphertext bits (one rounding
 * instead of three); the CPU oracle implements the same arithmetic (Evaluator::assemble_rot).  s1, s2 must be
 * non-zero rotations.  hb_assemble_hoisted takes the digits of `a` from hb_decompose.  No counterpart in HEaaN. */
int hb_assemble_rot(hb_ctx *ctx, const hb_ct *a, int64_t s1, const hb_pt *p1, int64_t s2, const hb_pt *p2, hb_ct **out);
int hb_assemble_hoisted(hb_ctx *ctx, const hb_ct *a, const hb_digits *digits, int64_t s1, const hb_pt *p1, int64_t s2, const hb_pt *p2,
                        hb_ct **out);
/* The same with the masks folded into the switching keys once.  mask (.) sum_dg digit_dg (.) key_dg equals
 * sum_dg digit_dg (.) (mask (.) key_dg) modulo every prime, so hb_masked_key_create(steps, m1, m2) stores
 * (m1 + m2) (.) key_steps restricted to the masks' level (m2 may be NULL), and hb_assemble_masked(a, digits, k1, k2)
 * gives exactly the residues of hb_assemble_hoisted(a, digits, s1, m1, s2, m2) with one inner product and one
 * reduction per residue (k2 may be NULL: a single masked rotation, e.g. when both steps are the same rotation and
 * the key carries m1 + m2).  A masked key is as large as nd * 2 * (level + 1 + K) limbs.  No counterpart in HEaaN. */
int hb_masked_key_create(hb_ctx *ctx, int64_t left_steps, const hb_pt *m1, const hb_pt *m2, hb_mkey **out);
void hb_masked_key_free(hb_mkey *key);
int hb_assemble_masked(hb_ctx *ctx, const hb_ct *a, const hb_digits *digits, const hb_mkey *k1, const hb_mkey *k2, hb_ct **out);
/* `groups` wrapped copies of the same input in one launch sequence: copy g uses k1s[g] and k2s[g] (k2s, or single
 * entries of it, may be NULL).  `out` holds groups * batch(a) members, member g * batch(a) + b = copy g of input b,
 * each bit for bit what hb_assemble_masked gives.  At most 16 groups.  Several iterations of a shift loop at once,
 * for batches too small to fill the GPU on their own. */
int hb_assemble_masked_multi(hb_ctx *ctx, const hb_ct *a, const hb_digits *digits, const hb_mkey *const *k1s, const hb_mkey *const *k2s,
                             int groups, hb_ct **out);
/* raw forward / inverse NTT of every limb of the batch, in place (primitive sweep) */
int hb_ntt(hb_ctx *ctx, hb_ct *a, int inverse);

/* Fused forms used by the matmul schedules (bit-identical to the unfused sequences). */
/* out = rescale(a (.) pa + b (.) pb)   -- MatrixUtils.cpp:1424-1427 "assemble" */
int hb_mul2_add_rescale(hb_ctx *ctx, const hb_ct *a, const hb_pt *pa, const hb_ct *b, const hb_pt *pb, hb_ct **out);
/* out = sum_j mult(a[j], p[j])  (each product rescaled, then added) -- the baby-step sums of the linear
 * transforms, MatrixUtils.cpp:815-823, 832-840.  At most 24 terms. */
int hb_mul_pt_sum(hb_ctx *ctx, const hb_ct *const *a, const hb_pt *const *p, int count, hb_ct **out);
/* out_g = rescale(sum_j multWithoutRescale(a[j], p[g * count + j])) for g < parts, all parts in one pass over the a[j]
 * (null plaintexts are skipped; at most 17 terms and 17 parts): the giant-step parts of a baby-step / giant-step
 * transform (MatrixUtils.cpp:776-1070) share their baby-step rotations.  out holds parts * batch members, part-major;
 * every part has the residues hb_sum_mul_pt_rescale gives for its terms. */
int hb_mul_pt_sum_parts(hb_ctx *ctx, const hb_ct *const *a, const hb_pt *const *p, int count, int parts, hb_ct **out);
/* out = rescale(sum_j a[j] (.) p[j]): the products are added un-rescaled and the sum is rescaled once (one inverse
 * transform of the last limb instead of one per term).  The masked sums of the linear transforms in schedule 2. */
int hb_sum_mul_pt_rescale(hb_ctx *ctx, const hb_ct *const *a, const hb_pt *const *p, int count, hb_ct **out);
/* acc += tensor(a, b); *acc may be NULL on entry -- MatrixUtils.cpp:1434-1439 */
int hb_tensor_acc(hb_ctx *ctx, const hb_ct *a, const hb_ct *b, hb_ct **acc);
/* *acc (+)= sum over g < groups of tensor(a[g], b[g]); a and b hold groups * batch members (group-major), *acc holds
 * batch members (NULL: created).  Same residues as `groups` calls of hb_tensor_acc. */
int hb_tensor_acc_groups(hb_ctx *ctx, const hb_ct *a, const hb_ct *b, int groups, hb_ct **acc);
/* out = sum_k pre[k] (.) rot_rows(pt, k * row_step), un-rescaled -- HomEvaluator::matmul :595-601 */
int hb_matmul_acc(hb_ctx *ctx, const hb_ct *pre, const hb_pt *pt, int64_t row_step, hb_ct **out);
/* the same over several K-groups at once: `pre` holds the shifted copies of `btotal` independent inputs, copy k of
 * input b at batch position k*btotal + b; the products of inputs b0 .. b0+bcount-1 with pts[0..bcount-1] are
 * summed into one ciphertext (matMulReUse + addInplace over groups, bert-matmul.cpp:262-268) */
int hb_matmul_acc_multi(hb_ctx *ctx, const hb_ct *pre, int btotal, int b0, const hb_pt *const *pts, int bcount, int64_t row_step, hb_ct **out);
/* The same for `tiles` outputs that share the shifted copies (all output tiles of a sublayer multiply the same copies of x):
 * out[t] = sum over b of matmul(copies of input b0 + b, pts[t * bcount + b]); the copies are read once per four tiles. */
int hb_matmul_acc_tiles(hb_ctx *ctx, const hb_ct *pre, int btotal, int b0, const hb_pt *const *pts, int bcount, int tiles, int64_t row_step,
                        hb_ct **out);
/* rotation of a plaintext (pure slot permutation, no key) -- leftRotate(ptxt) used at MatrixUtils.cpp:1503 */
int hb_pt_rotate(hb_ctx *ctx, const hb_pt *p, int64_t left_steps, hb_pt **out);
/* mult(ptxt, ptxt) with rescale and add(ptxt, ptxt), as multMatMat<Plaintext> uses them -- MatrixUtils.cpp:1556-1558 */
int hb_pt_mul(hb_ctx *ctx, const hb_pt *a, const hb_pt *b, hb_pt **out);
int hb_pt_add(hb_ctx *ctx, const hb_pt *a, const hb_pt *b, hb_pt **out);
/* modReduct after a lazy sum across ranks -- HomEvaluator.hpp:602-605 */
int hb_mod_reduce(hb_ctx *ctx, hb_ct *a);

/* Multi-GPU: sum (or gather) ciphertext tiles across ranks.  The communicator is created by the
 * caller (ncclComm_t passed as void*); replaces HEMMer::ncclAllReduceWrapper (HEMMer.cpp:2625-2635)
 * and TransformerBlock::ncclReduceWrapper* (TransformerBlock.cpp:11100-11154). */
/* communicator set-up: ncclGetUniqueId + ncclCommInitRank as in HEMMer.cpp:143-153 (the 128-byte id
 * travels between ranks by whatever channel the launcher has; the reference uses MPI_Bcast) */
int hb_nccl_unique_id(void *id128);
int hb_nccl_comm_init(hb_ctx *ctx, int nranks, int rank, const void *id128, void **comm);
int hb_nccl_comm_destroy(void *comm);
/* in place: a <- (sum over ranks of a) mod q on every rank -- HEMMer::ncclAllReduceWrapper (HEMMer.cpp:2625-2635) + modReduct */
int hb_allreduce_sum(hb_ctx *ctx, hb_ct *a, void *nccl_comm);
/* sum to one owner: on `root`, a <- (sum over ranks of a) mod q; elsewhere a is left as it was --
 * TransformerBlock::ncclReduceWrapper / ncclReduceWrapperHidden (TransformerBlock.cpp:11100-11140) + modReduct */
int hb_reduce_sum(hb_ctx *ctx, hb_ct *a, int root, int my_rank, void *nccl_comm);
/* `all` (batch = ranks * batch(mine)) receives every rank's `mine`, rank-major: tiles of a sublayer replicated for the next one */
int hb_allgather(hb_ctx *ctx, const hb_ct *mine, hb_ct *all, void *nccl_comm);
/* Point-to-point moves of whole handles for a K-split exchange in which only the ranks that hold partial products of
 * a tile talk to its owner.  Sends and receives are issued between hb_nccl_group_start() and hb_nccl_group_end() on
 * both sides (ncclGroupStart / ncclGroupEnd as in TransformerBlock.cpp:11106-11119); hb_sum_mod_reduce then adds the
 * owner's own partial product and the received ones and reduces modulo every prime in one pass (at most 16 parts). */
int hb_nccl_group_start(void);
int hb_nccl_group_end(void);
int hb_send(hb_ctx *ctx, const hb_ct *a, int peer, void *nccl_comm);
int hb_recv(hb_ctx *ctx, hb_ct *a, int peer, void *nccl_comm);
int hb_sum_mod_reduce(hb_ctx *ctx, const hb_ct *const *parts, int count, hb_ct **out);

/* Host threads used by the encode / decode halves of hb_encrypt_many / hb_decrypt_many (0: every core, at most 32).
 * Several ranks on one host each take cores / ranks.  No counterpart in the reference (one process per GPU under mpirun). */
int hb_set_host_threads(hb_ctx *ctx, int n);

/* CUDA graph of a fixed sequence of calls on this context (no counterpart in the reference, which launches every
 * kernel from the host each time).  Calls made between hb_graph_begin and hb_graph_end are recorded instead of run;
 * hb_graph_launch replays them on the context's stream.  Device buffers come from the context's pool exactly as in
 * an unrecorded pass, so the recorded kernels use fixed addresses: keep the operand handles alive and update them
 * in place only, and keep the result handles of the recorded pass while the graph is in use -- every replay writes
 * its results there.  Whatever is made on first use (rotation keys, masks, masked keys, per-level plans) must exist
 * before recording: run the sequence once first.  Calls that wait for the stream or copy to / from the host
 * (encode, encrypt, decrypt, import, export, sync) return HB_E_ARG while recording. */
typedef struct hb_graph hb_graph;
int hb_graph_begin(hb_ctx *ctx);
int hb_graph_end(hb_ctx *ctx, hb_graph **out);
int hb_graph_launch(hb_ctx *ctx, hb_graph *graph);
uint64_t hb_graph_kernels(const hb_graph *graph); /* kernels recorded in the graph */
void hb_graph_free(hb_graph *graph);

#ifdef __cplusplus
}
#endif
#endif /* HEMMER_B200_H */
