"""Scenarios shared by the CPU (oracle-only) and GPU (CUDA vs oracle) tests.

Each scenario drives one library through the HEMMer call surface on seeded inputs and returns
``(exports, err)``: the raw ciphertext residues of every result (for bit-exact comparison between
libraries) and the max-abs difference between the decrypted results and the float64 computation.
"""
import numpy as np


def tile_dim(lib):
    return int(round((lib.slots // 2) ** 0.5))


def _mats(seed, d, n, lo=-1.0, hi=1.0):
    rng = np.random.default_rng(seed)
    return [rng.uniform(lo, hi, (d, d)) for _ in range(n)]


def sc_transforms(lib, H):
    d = tile_dim(lib)
    A, B = _mats(100, d, 2)
    a = H.encrypt2(A, B, nonce=1)
    s, t = H.sigma(a), H.tau(a)
    S, T = H.decrypt2(s), H.decrypt2(t)
    sig = lambda M: np.stack([np.roll(M[r], -r) for r in range(d)])
    tau = lambda M: np.stack([np.roll(M[:, c], -c) for c in range(d)], axis=1)
    err = max(np.abs(S[0] - sig(A)).max(), np.abs(S[1] - sig(B)).max(), np.abs(T[0] - tau(A)).max(), np.abs(T[1] - tau(B)).max())
    tr = H.encrypt2(A, B, nonce=2)
    H.transpose_inplace(tr)
    R = H.decrypt2(tr)
    err = max(err, np.abs(R[0] - A.T).max(), np.abs(R[1] - B.T).max())
    return [lib.ct_export(x.ct) for x in (s, t, tr)], err


def sc_ccmm_single_tile(lib, H, target=2):
    """Single ct x ct product: one d x d tile per ciphertext, half of the slots used."""
    d = tile_dim(lib)
    A, B = _mats(101, d, 2)
    a, b = H.encrypt(A, nonce=3), H.encrypt(B, nonce=4)
    c = H.single_cc_matmul(a, b, target)
    assert lib.ct_meta(c.ct)[0] == target
    return [lib.ct_export(c.ct)], np.abs(H.decrypt(c) - A @ B).max()


def sc_ccmm_two_tiles(lib, H, target=2):
    d = tile_dim(lib)
    A, A2, B, B2 = _mats(102, d, 4)
    a, b = H.encrypt2(A, A2, nonce=5), H.encrypt2(B, B2, nonce=6)
    c = H.single_cc_matmul(a, b, target)
    D = H.decrypt2(c)
    return [lib.ct_export(c.ct)], max(np.abs(D[0] - A @ B).max(), np.abs(D[1] - A2 @ B2).max())


def sc_pcmm_reuse(lib, H, target=2):
    """matMulPre + matMulReUse + repack_notBTS on four K-tiles and two output tiles (bert-matmul.cpp:251-293)."""
    d = tile_dim(lib)
    X = _mats(103, d, 4)
    rngw = np.random.default_rng(104)
    W = [[rngw.normal(0, 0.02, (d, d)) for _ in range(4)] for _ in range(2)]
    x01, x23 = H.encrypt2(X[0], X[1], nonce=7), H.encrypt2(X[2], X[3], nonce=8)
    packed = H.complex_packing(x01, x23)
    pre = H.matmul_pre(packed, target)
    assert lib.ct_meta(pre)[:3] == (target + 1, 2, d)
    outs = []
    for j in range(2):
        w = H.encode_diagonal_to_row4(*W[j], level=target + 1)
        outs.append(H.matmul_reuse(pre, w))
    exports = [lib.ct_export(pre)] + [lib.ct_export(o.ct) for o in outs]
    # semantic: 2*Re(out_j) left half + right half = sum_k X_k W_jk
    err = 0.0
    for j in range(2):
        z = lib.decrypt(outs[j].ct).reshape(d, 2 * d)
        got = 2 * (z[:, :d].real + z[:, d:].real)
        err = max(err, np.abs(got - sum(X[k] @ W[j][k] for k in range(4))).max())
    rp = H.repack_not_bts(outs[0], outs[1])
    exports.append(lib.ct_export(rp.ct))
    return exports, err


def sc_cc_reuse(lib, H, target=2):
    """matMulPre / matMulPreRev / matMulCCReUse: encrypted right operand with shared left shifts."""
    d = tile_dim(lib)
    A, A2, B, B2 = _mats(105, d, 4)
    a, b = H.encrypt2(A, A2, nonce=9), H.encrypt2(B, B2, nonce=10)
    pre = H.matmul_pre(a, target)
    tb = H.matmul_pre_rev(b, target)
    c = H.matmul_cc_reuse(pre, tb)
    assert lib.ct_meta(c.ct)[3] == 2  # relinearised, not rescaled
    z = lib.decrypt(c.ct).real.reshape(d, 2 * d)
    err = max(np.abs(z[:, :d] - A @ B).max(), np.abs(z[:, d:] - A2 @ B2).max())
    return [lib.ct_export(tb.ct), lib.ct_export(c.ct)], err


def sc_packed(lib, H, target=2):
    """complexPacking* + packedMatMul + repackCC on a pair of tiles (TransformerBlock.cpp:2474-2482 pattern)."""
    d = tile_dim(lib)
    A, A2, B, B2 = _mats(106, d, 4)
    a, b = H.encrypt2(A, A2, nonce=11), H.encrypt2(B, B2, nonce=12)
    H.complex_packing_inplace(a)
    H.complex_packing_row_inplace(b)
    c = H.packed_matmul(a, b, target)
    r = H.repack_cc(c)
    D = H.decrypt2(r)
    err = max(np.abs(D[0] - A @ B).max(), np.abs(D[1] - A2 @ B2).max())
    return [lib.ct_export(a.ct), lib.ct_export(b.ct), lib.ct_export(c.ct), lib.ct_export(r.ct)], err


def sc_packed_reuse(lib, H, target=2):
    """packedMatMulPre / PreRot / PreRev / CCReuse and splitInTwo (bert-matmul-backward.cpp:317-384 pattern)."""
    d = tile_dim(lib)
    A, A2, B, B2 = _mats(107, d, 4)
    a, b = H.encrypt2(A, A2, nonce=13), H.encrypt2(B, B2, nonce=14)
    H.complex_packing_inplace(a)
    H.complex_packing_row_inplace(b)
    sa = H.packed_matmul_pre(a, target)
    pre = H.packed_matmul_pre_rot(sa, target)
    tb = H.packed_matmul_pre_rev(b, target)
    c = H.packed_matmul_cc_reuse(pre, tb)
    r = H.repack_cc(c)
    D = H.decrypt2(r)
    err = max(np.abs(D[0] - A @ B).max(), np.abs(D[1] - A2 @ B2).max())
    s1, s2 = H.split_in_two(r)
    D1, D2 = H.decrypt2(s1), H.decrypt2(s2)
    err = max(err, np.abs(D1[0] - A @ B).max(), np.abs(D1[1] - A @ B).max(), np.abs(D2[0] - A2 @ B2).max(), np.abs(D2[1] - A2 @ B2).max())
    return [lib.ct_export(x) for x in (pre, tb.ct, c.ct, s1.ct, s2.ct)], err


def sc_transpose_packing(lib, H, target=0):
    d = tile_dim(lib)
    A, A2 = _mats(108, d, 2)
    a = H.encrypt2(A, A2, nonce=15)
    H.transpose_complex_packing_inplace(a, target)
    z = lib.decrypt(a.ct).reshape(d, 2 * d)
    # even columns keep value - i * (next column), then the transpose of each tile
    def fold(M):
        F = np.zeros((d, d), dtype=complex)
        F[:, 0::2] = M[:, 0::2] - 1j * M[:, 1::2]
        F[:, 1::2] = F[:, 0::2]
        return F.T
    err = max(np.abs(z[:, :d] - fold(A)).max(), np.abs(z[:, d:] - fold(A2)).max())
    b = H.encrypt2(A, A2, nonce=16)
    c = H.complex_packing_rev(b, b)
    zz = lib.decrypt(c.ct)
    base = np.concatenate([A, A2], axis=1).reshape(-1)
    err = max(err, np.abs(zz - (base - 1j * base)).max())
    return [lib.ct_export(a.ct), lib.ct_export(c.ct)], err


def sc_batched(lib, H, target=2):
    """Batched handles: three ct x ct products and two K-groups of ct x pt behind one launch sequence must give,
    entry by entry, the ciphertexts of the same calls made one at a time."""
    from importlib import import_module
    CtxtTensor = import_module("encryption-friendly_llm_architecture_b200").CtxtTensor
    d = tile_dim(lib)
    mats = _mats(109, d, 12)
    As = [H.encrypt2(mats[2 * k], mats[2 * k + 1], nonce=20 + k) for k in range(3)]
    Bs = [H.encrypt2(mats[6 + 2 * k], mats[7 + 2 * k], nonce=30 + k) for k in range(3)]
    def batch(cts):
        lvl, npoly, _, sp = lib.ct_meta(cts[0].ct)
        out = lib.ct_create(lvl, npoly, len(cts), sp)
        for k, c in enumerate(cts):
            lib.batch_set(out, k, c.ct)
        return CtxtTensor(out, *cts[0].shape)
    ab, bb = batch(As), batch(Bs)
    H.transpose_inplace(bb)
    cb = H.single_cc_matmul(ab, bb, target)
    exports = [lib.ct_export(cb.ct)]
    err = 0.0
    for k in range(3):
        bk = CtxtTensor(Bs[k].ct, *Bs[k].shape)
        H.transpose_inplace(bk)
        ck = H.single_cc_matmul(As[k], bk, target)
        assert np.array_equal(lib.ct_export(ck.ct)[0], exports[0][k]), "batched ct x ct differs from the single call"
        z = lib.decrypt(cb.ct, k)[: 2 * d * d].real.reshape(d, 2 * d)
        err = max(err, np.abs(z[:, :d] - mats[2 * k] @ mats[6 + 2 * k].T).max(), np.abs(z[:, d:] - mats[2 * k + 1] @ mats[7 + 2 * k].T).max())
    # the two-half form of the product (transforms per group, one product loop) gives the same ciphertexts
    sa, tb = H.cc_matmul_prepare(ab, bb, target)
    split = H.cc_matmul_core(sa, tb, d, d, d, 2 * d, target)
    assert np.array_equal(lib.ct_export(split.ct), exports[0]), "prepare + core differs from singleCCMatMul"
    # two K-groups through matMulPre as one batch, summed per output tile in one pass
    rngw = np.random.default_rng(110)
    W = [[rngw.normal(0, 0.02, (d, d)) for _ in range(4)] for _ in range(2)]
    pk = [H.complex_packing(As[0], As[1]), H.complex_packing(As[1], As[2])]
    pre_b = H.matmul_pre(batch(pk), target)
    wts = [H.encode_diagonal_to_row4(*W[g], level=target + 1) for g in range(2)]
    fused = H.matmul_reuse_groups(pre_b, 2, 0, wts)
    singles = [H.matmul_reuse(H.matmul_pre(pk[g], target), wts[g]) for g in range(2)]
    ref = lib.add(singles[0].ct, singles[1].ct)
    assert np.array_equal(lib.ct_export(fused.ct), lib.ct_export(ref)), "fused K-group sum differs from matMulReUse + addInplace"
    exports.append(lib.ct_export(fused.ct))
    return exports, err


def sc_single_matmul(lib, H, target=2):
    """HEMMer::singleMatMul (ct x pt without reuse) on two side-by-side tiles, plus the plaintext primitives it uses."""
    d = tile_dim(lib)
    A, A2 = _mats(111, d, 2)
    rngw = np.random.default_rng(112)
    W, W2 = rngw.normal(0, 0.02, (d, d)), rngw.normal(0, 0.02, (d, d))
    a = H.encrypt2(A, A2, nonce=40)
    w = H.encode2(W, W2, level=target + 3)
    c = H.single_matmul(a, w, target)
    assert lib.ct_meta(c.ct)[0] == target
    D = H.decrypt2(c)
    err = max(np.abs(D[0] - A @ W).max(), np.abs(D[1] - A2 @ W2).max())
    z = np.random.default_rng(113).uniform(-1, 1, lib.slots)
    p1, p2 = lib.encode(z, 4), lib.encode(z[::-1].copy(), 4)
    prod, summ, rot = lib.pt_mul(p1, p2), lib.pt_add(p1, p2), lib.pt_rotate(p1, 5)
    err = max(err, np.abs(lib.decode(prod).real - z * z[::-1]).max(), np.abs(lib.decode(summ).real - (z + z[::-1])).max(),
              np.abs(lib.decode(rot).real - np.roll(z, -5)).max())
    return [lib.ct_export(c.ct), lib.pt_export(prod)[None, None], lib.pt_export(summ)[None, None], lib.pt_export(rot)[None, None]], err


def _thin_cols(M, d, r):
    """[T0 | T1]: the d x r row block k of M sits in columns [r (k // 2), r (k // 2) + r) of tile k % 2."""
    T = [np.zeros((d, d)), np.zeros((d, d))]
    for k in range(M.shape[0] // d):
        T[k % 2][:, r * (k // 2):r * (k // 2) + r] = M[k * d:(k + 1) * d]
    return T


def _thin_rows(M, d, r):
    """[T0 | T1]: the r x d column block k of M sits in rows [r (k // 2), r (k // 2) + r) of tile k % 2."""
    T = [np.zeros((d, d)), np.zeros((d, d))]
    for k in range(M.shape[1] // d):
        T[k % 2][r * (k // 2):r * (k // 2) + r, :] = M[:, k * d:(k + 1) * d]
    return T


def _pairs(H, M, d, nonce):
    return [H.encrypt2(M[:, 2 * i * d:(2 * i + 1) * d].copy(), M[:, (2 * i + 1) * d:(2 * i + 2) * d].copy(), nonce=nonce + i) for i in range(M.shape[1] // (2 * d))]


def sc_lora_forward(lib, H, target=4, r=2):
    """The LoRA branch of a projection as the reference runs it (TransformerBlock.cpp:1787-1835, without the
    bootstraps): X Wa by matMulHighLow on three tile pairs, repackToOneCol, then (X Wa) Wb by matMulLowLow."""
    d = tile_dim(lib)
    rng = np.random.default_rng(120)
    X, Wa, Wb = rng.uniform(-1, 1, (d, 6 * d)), rng.normal(0, 0.2, (6 * d, r)), rng.normal(0, 0.2, (r, 6 * d))
    cur = _pairs(H, X, d, 50)
    lora_wa, lora_wb = H.encrypt2(*_thin_cols(Wa, d, r), nonce=56), H.encrypt2(*_thin_rows(Wb, d, r), nonce=57)
    acc = None
    for i in range(3):
        part = H.matmul_high_low(cur[i], H.get_low_col_block(lora_wa, i, r), i, target, r)
        if acc is None:
            acc = part
        else:
            H.add_inplace(acc, part)
    assert lib.ct_meta(acc.ct)[0] == target
    xa = H.repack_to_one_col(acc, 0, r)
    z = lib.decrypt(xa.ct).real.reshape(d, 2 * d)
    want = np.zeros((d, 2 * d))
    want[:, :r] = want[:, d:d + r] = X @ Wa
    err = np.abs(z - want).max()
    exports = [lib.ct_export(acc.ct), lib.ct_export(xa.ct)]
    t2 = lib.ct_meta(xa.ct)[0] - 3
    for i in range(3):
        out = H.matmul_low_low(xa, H.get_low_row_block(lora_wb, i, r), 0, i, t2, r)
        z = lib.decrypt(out.ct).real.reshape(d, 2 * d)
        err = max(err, np.abs(z - (X @ Wa @ Wb)[:, 2 * i * d:(2 * i + 2) * d]).max())
        exports.append(lib.ct_export(out.ct))
    return exports, err


def sc_lora_backward(lib, H, target=4, r=2):
    """Gradients of the two LoRA factors (TransformerBlock.cpp:10500-10535): (X Wa)^T dY by matMulLowHigh +
    repackToMultiRow, X^T (dY Wb^T) by matMulHighLow + repackToMultiCol; and repackToOneRow on its own."""
    d = tile_dim(lib)
    rng = np.random.default_rng(121)
    X, dY = rng.uniform(-1, 1, (d, 6 * d)), rng.uniform(-1, 1, (d, 6 * d))
    XA, G = rng.uniform(-1, 1, (d, r)), rng.uniform(-1, 1, (d, r))  # stand-ins for X Wa and dY Wb^T
    dYc = _pairs(H, dY, d, 60)
    P = np.zeros((d, d)); P[:r, :] = XA.T
    Q = np.zeros((d, d)); Q[:, :r] = G
    in_b, gb = H.encrypt2(P, P, nonce=66), H.encrypt2(Q, Q, nonce=67)
    grad_wb = grad_wa = None
    for i in range(3):
        m = H.repack_to_multi_row(H.matmul_low_high(in_b, dYc[i], 0, target, r), i, r)
        if grad_wb is None:
            grad_wb = m
        else:
            H.add_inplace(grad_wb, m)
        xt = H.encrypt2(X[:, 2 * i * d:(2 * i + 1) * d].T.copy(), X[:, (2 * i + 1) * d:(2 * i + 2) * d].T.copy(), nonce=70 + i)
        m = H.repack_to_multi_col(H.matmul_high_low(xt, gb, 0, target, r), i, r)
        if grad_wa is None:
            grad_wa = m
        else:
            H.add_inplace(grad_wa, m)
    z = lib.decrypt(grad_wb.ct).real.reshape(d, 2 * d)
    err = np.abs(z - np.concatenate(_thin_rows(XA.T @ dY, d, r), axis=1)).max()
    z = lib.decrypt(grad_wa.ct).real.reshape(d, 2 * d)
    want = np.concatenate(_thin_cols(np.concatenate([X[:, k * d:(k + 1) * d].T @ G for k in range(6)]), d, r), axis=1)
    err = max(err, np.abs(z - want).max())
    # repackToOneRow: every r-row band of both tiles summed into band `block` of both tiles
    M = rng.uniform(-1, 1, (d, 2 * d))
    blk = 1
    one = H.repack_to_one_row(H.encrypt2(M[:, :d].copy(), M[:, d:].copy(), nonce=75), blk, r)
    band = sum(M[j:j + r, :d] + M[j:j + r, d:] for j in range(0, d, r))
    want = np.zeros((d, 2 * d))
    want[blk * r:(blk + 1) * r, :d] = want[blk * r:(blk + 1) * r, d:] = band
    err = max(err, np.abs(lib.decrypt(one.ct).real.reshape(d, 2 * d) - want).max())
    return [lib.ct_export(grad_wb.ct), lib.ct_export(grad_wa.ct), lib.ct_export(one.ct)], err


def sc_repack_lora_opti(lib, H, target=2):
    """repack_loraOpti on two un-rescaled matMulReUse results, against the same slot arithmetic in the clear."""
    d = tile_dim(lib)
    X = _mats(122, d, 4)
    rngw = np.random.default_rng(123)
    x01, x23 = H.encrypt2(X[0], X[1], nonce=80), H.encrypt2(X[2], X[3], nonce=81)
    pre = H.matmul_pre(H.complex_packing(x01, x23), target)
    outs = [H.matmul_reuse(pre, H.encode_diagonal_to_row4(*[rngw.normal(0, 0.05, (d, d)) for _ in range(4)], level=target + 1)) for _ in range(2)]
    rp = H.repack_lora_opti(outs[0], outs[1])
    u, v = lib.decrypt(outs[0].ct), lib.decrypt(outs[1].ct)
    out = 2 * u.real + 2j * v.real
    tmp = np.roll(out, -d)
    out = out + tmp
    conj = np.conj(out)
    out = out + conj
    tmp = 1j * (conj - tmp)
    m = np.zeros(lib.slots)
    m.reshape(-1, 2 * d)[:d, :d] = 0.5
    want = m * out + np.roll(m * tmp, d)
    return [lib.ct_export(rp.ct)], np.abs(lib.decrypt(rp.ct) - want).max()


def sc_rot_sum_hadamard(lib, H, target=0):
    """oneMatRotSumInplace (HEMMer.cpp:882-919) and hadamardMultInplace with a ciphertext and with a plaintext operand."""
    d = tile_dim(lib)
    A, A2, B, B2 = _mats(130, d, 4)
    a, b = H.encrypt2(A, A2, nonce=90), H.encrypt2(B, B2, nonce=91)
    H.one_mat_rot_sum_inplace(a, b)
    Da, Db = H.decrypt2(a), H.decrypt2(b)
    half = d // 2
    bc = lambda M: np.repeat(M.sum(axis=1, keepdims=True), d, axis=1)
    err = max(np.abs(Da[0] - bc(A[:, :half])).max(), np.abs(Da[1] - bc(A2[:, :half])).max(),
              np.abs(Db[0] - bc(B[:, half:])).max(), np.abs(Db[1] - bc(B2[:, half:])).max())
    x, y = H.encrypt2(A, A2, nonce=92), H.encrypt2(B, B2, nonce=93)
    H.hadamard_mult_inplace(x, y)
    Dx = H.decrypt2(x)
    err = max(err, np.abs(Dx[0] - A * B).max(), np.abs(Dx[1] - A2 * B2).max())
    z = H.encrypt2(A, A2, nonce=94)
    H.hadamard_mult_inplace(z, H.encode2(B, B2))
    Dz = H.decrypt2(z)
    err = max(err, np.abs(Dz[0] - A * B).max(), np.abs(Dz[1] - A2 * B2).max())
    return [lib.ct_export(t.ct) for t in (a, b, x, z)], err


def sc_tr_rot_sum(lib, H, target=2):
    """tr_oneMatRotSumInplace (HEMMer.cpp:921-962): level-down, sums over a whole tile row, result on half of the row."""
    d = tile_dim(lib)
    A, A2, B, B2 = _mats(133, d, 4)
    a, b = H.encrypt2(A, A2, nonce=96), H.encrypt2(B, B2, nonce=97)
    H.tr_one_mat_rot_sum_inplace(a, b, target)
    assert lib.ct_meta(a.ct)[0] == target and lib.ct_meta(b.ct)[0] == target
    Da, Db = H.decrypt2(a), H.decrypt2(b)
    half = d // 2

    def want(M, left):
        out = np.zeros((d, d))
        s = M.sum(axis=1, keepdims=True)
        if left:
            out[:, :half] = s
        else:
            out[:, half:] = s
        return out
    err = max(np.abs(Da[0] - want(A, True)).max(), np.abs(Da[1] - want(A2, True)).max(),
              np.abs(Db[0] - want(B, False)).max(), np.abs(Db[1] - want(B2, False)).max())
    return [lib.ct_export(t.ct) for t in (a, b)], err


def sc_masks_and_sums(lib, H, target=0):
    """maskFirstCol / maskLeftHalf / maskRightHalf (HEMMer.cpp:1251-1269), squareSum (:2499-2510) and
    reduceRowSumWithScaledMask (:2512-2530, one rank) on two side-by-side tiles."""
    d = tile_dim(lib)
    A, A2, B, B2 = _mats(134, d, 4)
    exports, err = [], 0.0
    for k, (fn, keep) in enumerate(((H.mask_first_col_inplace, lambda r, c: c % d == 0), (H.mask_left_half_inplace, lambda r, c: c < d),
                                    (H.mask_right_half_inplace, lambda r, c: c >= d))):
        x = H.encrypt2(A, A2, nonce=98 + k)
        fn(x)
        D = H.decrypt2(x)
        full = np.concatenate([A, A2], axis=1)
        want = np.array([[full[r, c] if keep(r, c) else 0.0 for c in range(2 * d)] for r in range(d)])
        err = max(err, np.abs(np.concatenate([D[0], D[1]], axis=1) - want).max())
        exports.append(lib.ct_export(x.ct))
    xs = [H.encrypt2(A, A2, nonce=110), H.encrypt2(B, B2, nonce=111), H.encrypt2(0.5 * A, 0.5 * B2, nonce=112)]
    sq = H.square_sum(xs)
    D = H.decrypt2(sq)
    err = max(err, np.abs(D[0] - (A * A + B * B + 0.25 * A * A)).max(), np.abs(D[1] - (A2 * A2 + B2 * B2 + 0.25 * B2 * B2)).max())
    exports.append(lib.ct_export(sq.ct))
    y = H.encrypt2(A, A2, nonce=113)
    scaled = np.zeros((d, d)); scaled[:, 0] = 1.0 / d
    H.reduce_row_sum_with_scaled_mask(y, H.encode2(scaled, np.zeros((d, d)), level=lib.ct_meta(y.ct)[0]))
    D = H.decrypt2(y)
    # row sums over the 2d-wide row, gathered at the first column and spread back over the row: every entry of a row
    # holds the mean over the d columns of tile 0 plus the d columns of tile 1, divided by d
    row = (A.sum(axis=1) + A2.sum(axis=1)) / d
    err = max(err, np.abs(D[0] - row[:, None]).max(), np.abs(D[1] - row[:, None]).max())
    exports.append(lib.ct_export(y.ct))
    return exports, err


def sc_lora_opti(lib, H, target=0):
    """The rank-2 LoRA branch of the reference's attention layer (TransformerBlock.cpp:2199-2365): X A B by slot-wise
    products and rotate-and-add, factors packed one rank vector per row."""
    d = tile_dim(lib)
    rng = np.random.default_rng(131)
    X, Wa, Wb = rng.uniform(-1, 1, (d, 6 * d)), rng.normal(0, 0.2, (6 * d, 2)), rng.normal(0, 0.2, (2, 6 * d))
    cur = _pairs(H, X, d, 95)
    fa, fb = np.zeros((d, 2 * d)), np.zeros((d, 2 * d))
    for i in range(3):
        for j in range(2):
            fa[2 * i + j] = Wa[2 * d * i:2 * d * (i + 1), j]
            fb[2 * i + j] = Wb[j, 2 * d * i:2 * d * (i + 1)]
    wa, wb = H.encrypt2(fa[:, :d].copy(), fa[:, d:].copy(), nonce=98), H.encrypt2(fb[:, :d].copy(), fb[:, d:].copy(), nonce=99)
    outs = H.lora_opti_forward(cur, wa, wb)
    want = X @ Wa @ Wb
    err = 0.0
    for i, o in enumerate(outs):
        z = lib.decrypt(o.ct).real.reshape(d, 2 * d)
        err = max(err, np.abs(z - want[:, 2 * d * i:2 * d * (i + 1)]).max())
    return [lib.ct_export(o.ct) for o in outs], err


def sc_gaussian_kernel(lib, H, target=2):
    """Score assembly of the reference's Gaussian-kernel attention (TransformerBlock.cpp:2420-2482): squared distances
    between query and key rows, per head (two heads per tile, two tiles per ciphertext), with chained levels."""
    d = tile_dim(lib)
    Q, Q2, K, K2 = _mats(132, d, 4, -0.5, 0.5)
    q, k = H.encrypt2(Q, Q2, nonce=100), H.encrypt2(K, K2, nonce=101)
    outs = H.gaussian_kernel_scores(q, k, target)
    err = 0.0
    half = d // 2
    for j, o in enumerate(outs):
        assert lib.ct_meta(o.ct)[0] == target
        D = H.decrypt2(o)
        for t, (A, B) in enumerate(((Q, K), (Q2, K2))):
            a, b = A[:, j * half:(j + 1) * half], B[:, j * half:(j + 1) * half]
            want = (a * a).sum(1)[:, None] + (b * b).sum(1)[None, :] - 2 * a @ b.T
            err = max(err, np.abs(D[t] - want).max())
    return [lib.ct_export(o.ct) for o in outs], err


SCENARIOS = {
    "masks_and_sums": sc_masks_and_sums,
    "tr_rot_sum": sc_tr_rot_sum,
    "gaussian_kernel": sc_gaussian_kernel,
    "lora_opti": sc_lora_opti,
    "rot_sum_hadamard": sc_rot_sum_hadamard,
    "repack_lora_opti": sc_repack_lora_opti,
    "lora_forward": sc_lora_forward,
    "lora_backward": sc_lora_backward,
    "single_matmul": sc_single_matmul,
    "batched": sc_batched,
    "transforms": sc_transforms,
    "ccmm_single_tile": sc_ccmm_single_tile,
    "ccmm_two_tiles": sc_ccmm_two_tiles,
    "pcmm_reuse": sc_pcmm_reuse,
    "cc_reuse": sc_cc_reuse,
    "packed": sc_packed,
    "packed_reuse": sc_packed_reuse,
    "transpose_packing": sc_transpose_packing,
}
