"""Python mirror of the HELLM::HEMMer call surface (ciphertext/include/HELLM/HEMMer.hpp).

Every method forwards to the native ``hb_hemmer_*`` entry points (C++ schedules over the
CUDA C ABI).  The only Python-side work is laying matrices out into slot vectors the way
``HEMMer::encode`` / ``encode2`` / ``msgDiagonalToRow4`` do (HEMMer.cpp:232-275, 353-398)
when a caller prefers to hand in numpy arrays.
"""
from __future__ import annotations

import ctypes as C
import numpy as np

from .capi import Handle, Lib, HBError


class CtxtTensor:
    """HETensor<Ciphertext> (HETensor.hpp:46-86): a ciphertext handle plus its tile shape."""

    def __init__(self, ct: Handle, rows: int, cols: int, width: int | None = None):
        if width is None:
            width = 1
            while cols > width:
                width <<= 1
        self.ct, self.rows, self.cols, self.width = ct, rows, cols, width

    @property
    def shape(self):
        return (self.rows, self.cols, self.width)


class PtxtTensor(CtxtTensor):
    """HETensor<Plaintext>."""


# ---- slot layouts (pure data movement) ----
def layout1(m, slots):
    """HEMMer::encode: row-major copy into the first rows*cols slots."""
    v = np.zeros(slots, dtype=np.complex128)
    v[: m.size] = np.asarray(m).reshape(-1)
    return v


def layout2(a, b, slots):
    """HEMMer::message2: [A | B] concatenated on columns."""
    return layout1(np.concatenate([a, b], axis=1), slots)


def layout_diag_to_row4(w1, w2, w3, w4, slots):
    """HEMMer::msgDiagonalToRow4: 1/2 (W1 - i W3) | 1/2 (W2 - i W4), column j rolled up by j."""
    left = 0.5 * (np.asarray(w1, dtype=np.float64) - 1j * np.asarray(w3, dtype=np.float64))
    right = 0.5 * (np.asarray(w2, dtype=np.float64) - 1j * np.asarray(w4, dtype=np.float64))
    for j in range(1, left.shape[1]):
        left[:, j] = np.roll(left[:, j], -j)
        right[:, j] = np.roll(right[:, j], -j)
    return layout1(np.concatenate([left, right], axis=1), slots)


class Hemmer:
    def __init__(self, lib: Lib, dll: C.CDLL | None = None, prefix: str | None = None):
        self.lib = lib
        self.dll = dll if dll is not None else lib.dll
        self.prefix = prefix if prefix is not None else lib.prefix + "hemmer_"
        self.h = C.c_void_p()
        self._fn("destroy").restype = None
        rc = self._fn("create")(lib.ctx, C.byref(self.h))
        if rc != 0:
            raise HBError(rc, "hemmer_create failed")
        self._nonce = 1000
        self.schedule = 0

    def _fn(self, name):
        return getattr(self.dll, self.prefix + name)

    def set_schedule(self, mode: int):
        """0: the reference's rotation sequence (default); 1: direct rotations of the transformed operand, hoisted;
        2: as 1, with each wrapped copy of the shift loops made by one assemble_rot (one division by P * q_level)."""
        self.lib._chk(self._fn("set_schedule")(self.h, C.c_int(mode)))
        self.schedule = mode

    def close(self):
        if self.h:
            self._fn("destroy")(self.h)
            self.h = C.c_void_p()

    def _call(self, name, *args, n_out=1):
        outs = [C.c_void_p() for _ in range(n_out)]
        rc = self._fn(name)(self.h, *args, *[C.byref(o) for o in outs])
        if rc != 0 and hasattr(self.dll, self.prefix + "last_error"):
            f = self._fn("last_error")
            f.restype = C.c_char_p
            raise HBError(rc, f().decode())
        self.lib._chk(rc)
        hs = [Handle(self.lib, o, "ct") for o in outs]
        return hs[0] if n_out == 1 else hs

    @staticmethod
    def _shp(t):
        return (C.c_int(t.rows), C.c_int(t.cols), C.c_int(t.width))

    # ---- encode / encrypt / decrypt (HEMMer.hpp:65-98) ----
    def next_nonce(self):
        self._nonce += 1
        return self._nonce

    def _native(self, name):
        """The library's own entry point for a HEMMer method that takes host matrices, when it has one (the CUDA library's
        C++ layer does; a library that only exports the tile schedules gets the layout done here)."""
        return getattr(self.dll, self.prefix + name, None)

    @staticmethod
    def _mat(m):
        a = np.ascontiguousarray(m, dtype=np.float64)
        return a, a.ctypes.data_as(C.POINTER(C.c_double))

    def _native_out(self, fn, kind, *args):
        out = C.c_void_p()
        rc = fn(self.h, *args, C.byref(out))
        if rc != 0:
            f = self._fn("last_error")
            f.restype = C.c_char_p
            raise HBError(rc, f().decode())
        return Handle(self.lib, out, kind)

    def encode(self, data, level=0):
        fn = self._native("encode")
        if fn is None:
            level = level or self.lib.L
            return PtxtTensor(self.lib.encode(layout1(data, self.lib.slots), level), data.shape[0], data.shape[1])
        a, pa = self._mat(data)
        return PtxtTensor(self._native_out(fn, "pt", pa, C.c_int(a.shape[0]), C.c_int(a.shape[1]), C.c_int(level)), a.shape[0], a.shape[1])

    def encode2(self, d1, d2, level=0):
        fn = self._native("encode2")
        if fn is None:
            level = level or self.lib.L
            return PtxtTensor(self.lib.encode(layout2(d1, d2, self.lib.slots), level), d1.shape[0], d1.shape[1], 2 * d1.shape[1])
        (a, pa), (b, pb) = self._mat(d1), self._mat(d2)
        return PtxtTensor(self._native_out(fn, "pt", pa, pb, C.c_int(a.shape[0]), C.c_int(a.shape[1]), C.c_int(level)), a.shape[0], a.shape[1], 2 * a.shape[1])

    def encode_diagonal_to_row4(self, w1, w2, w3, w4, level=0):
        fn = self._native("encode_diagonal_to_row4")
        if fn is None:
            level = level or self.lib.L
            return PtxtTensor(self.lib.encode(layout_diag_to_row4(w1, w2, w3, w4, self.lib.slots), level),
                              w1.shape[0], w1.shape[1], 2 * w1.shape[1])
        ms = [self._mat(w) for w in (w1, w2, w3, w4)]
        a = ms[0][0]
        return PtxtTensor(self._native_out(fn, "pt", *[p for _, p in ms], C.c_int(a.shape[0]), C.c_int(a.shape[1]), C.c_int(level)),
                          a.shape[0], a.shape[1], 2 * a.shape[1])

    def encrypt(self, data, nonce=None):
        nonce = self.next_nonce() if nonce is None else nonce
        fn = self._native("encrypt")
        if fn is None:
            pt = self.encode(data)
            return CtxtTensor(self.lib.encrypt(pt.ct, nonce), pt.rows, pt.cols, pt.width)
        a, pa = self._mat(data)
        return CtxtTensor(self._native_out(fn, "ct", pa, C.c_int(a.shape[0]), C.c_int(a.shape[1]), C.c_uint64(nonce)), a.shape[0], a.shape[1])

    def encrypt2(self, d1, d2, nonce=None):
        nonce = self.next_nonce() if nonce is None else nonce
        fn = self._native("encrypt2")
        if fn is None:
            pt = self.encode2(d1, d2)
            return CtxtTensor(self.lib.encrypt(pt.ct, nonce), pt.rows, pt.cols, pt.width)
        (a, pa), (b, pb) = self._mat(d1), self._mat(d2)
        return CtxtTensor(self._native_out(fn, "ct", pa, pb, C.c_int(a.shape[0]), C.c_int(a.shape[1]), C.c_uint64(nonce)), a.shape[0], a.shape[1], 2 * a.shape[1])

    def encrypt2_many(self, pairs, nonces):
        """encrypt2 for a list of (left, right) tile pairs: one batched CtxtTensor, member i = encrypt2(*pairs[i], nonces[i])."""
        msgs = np.stack([layout2(a, b, self.lib.slots).real for a, b in pairs])
        d = pairs[0][0].shape
        return CtxtTensor(self.lib.encrypt_many(msgs, self.lib.L, nonces), d[0], d[1], 2 * d[1])

    def decrypt(self, t):
        fn = self._native("decrypt")
        if fn is None:
            z = self.lib.decrypt(t.ct)
            return z[: t.rows * t.cols].real.reshape(t.rows, t.cols)
        out = np.zeros((t.rows, t.cols))
        self.lib._chk(fn(self.h, t.ct.ptr, *self._shp(t), out.ctypes.data_as(C.POINTER(C.c_double))))
        return out

    def decrypt2(self, t):
        fn = self._native("decrypt2")
        if fn is None:
            z = self.lib.decrypt(t.ct)[: t.rows * 2 * t.cols].real.reshape(t.rows, 2 * t.cols)
            return np.stack([z[:, : t.cols], z[:, t.cols:]])
        out = np.zeros((2, t.rows, t.cols))
        self.lib._chk(fn(self.h, t.ct.ptr, *self._shp(t), out.ctypes.data_as(C.POINTER(C.c_double))))
        return out

    def hadamard_mult_inplace(self, a, b):
        """HEMMer::hadamardMultInplace: slot-wise product with a ciphertext tensor or a plaintext tensor."""
        name = "hadamard_mult_pt" if isinstance(b, PtxtTensor) else "hadamard_mult"
        a.ct = self._call(name, a.ct.ptr, b.ct.ptr)

    def mask_first_col_inplace(self, t):
        t.ct = self._call("mask_inplace", t.ct.ptr, C.c_int(0), *self._shp(t))

    def mask_left_half_inplace(self, t):
        t.ct = self._call("mask_inplace", t.ct.ptr, C.c_int(1), *self._shp(t))

    def mask_right_half_inplace(self, t):
        t.ct = self._call("mask_inplace", t.ct.ptr, C.c_int(2), *self._shp(t))

    def square_sum(self, tensors):
        """HEMMer::squareSum (HEMMer.cpp:2499-2510): sum of the squares with one relinearisation and one rescale."""
        arr = (C.c_void_p * len(tensors))(*[t.ct.ptr.value for t in tensors])
        return CtxtTensor(self._call("square_sum", arr, C.c_int(len(tensors)), *self._shp(tensors[0])), *tensors[0].shape)

    def reduce_row_sum_with_scaled_mask(self, t, mask):
        """HEMMer::reduceRowSumWithScaledMask (HEMMer.cpp:2512-2530) on one rank; mask: a plaintext tensor at t's level."""
        t.ct = self._call("reduce_row_sum_with_scaled_mask", t.ct.ptr, mask.ct.ptr, *self._shp(t))

    def tr_one_mat_rot_sum_inplace(self, a, b, target_level=0):
        """HEMMer::tr_oneMatRotSumInplace (HEMMer.cpp:921-962): row sums over the whole tile side, on half of the row."""
        a.ct, b.ct = self._call("tr_one_mat_rot_sum", a.ct.ptr, b.ct.ptr, C.c_int(target_level), n_out=2)

    def gaussian_kernel_scores(self, query, key, target_level=4):
        """Score assembly of the reference's Gaussian-kernel attention (TransformerBlock.cpp:2420-2482) for one query / key
        pair: [|q_r|^2 + |k_c|^2 - 2 q_r . k_c] per head; returns the two head positions."""
        outs = self._call("gaussian_kernel_scores", query.ct.ptr, key.ct.ptr, *self._shp(query), C.c_int(target_level), n_out=2)
        return [CtxtTensor(o, *query.shape) for o in outs]

    def lora_opti_forward(self, cur, lora_wa, lora_wb):
        """The rank-2 LoRA branch of TransformerBlock::attention2_bert_loraOpti (TransformerBlock.cpp:2199-2365): three
        activation pairs and the two factor ciphertexts in, the three pairs of X A B out."""
        outs = self._call("lora_opti_forward", cur[0].ct.ptr, cur[1].ct.ptr, cur[2].ct.ptr, lora_wa.ct.ptr, lora_wb.ct.ptr, n_out=3)
        return [CtxtTensor(o, *cur[0].shape) for o in outs]

    def one_mat_rot_sum_inplace(self, a, b):
        """HEMMer::oneMatRotSumInplace: row sums of the left halves of a's tiles / right halves of b's, spread over the rows."""
        a.ct, b.ct = self._call("one_mat_rot_sum", a.ct.ptr, b.ct.ptr, n_out=2)

    # ---- matmul family ----
    def add_inplace(self, a, b):
        a.ct = self.lib.add(a.ct, b.ct)

    def single_cc_matmul(self, a, b, target_level=4):
        ct = self._call("matmul_cc", a.ct.ptr, *self._shp(a), b.ct.ptr, *self._shp(b), C.c_int(target_level))
        return CtxtTensor(ct, a.rows, b.cols, a.width)

    def single_matmul(self, a, b, target_level=4):
        """HEMMer::singleMatMul: ciphertext x plaintext without reuse."""
        ct = self._call("matmul_cp", a.ct.ptr, *self._shp(a), b.ct.ptr, *self._shp(b), C.c_int(target_level))
        return CtxtTensor(ct, a.rows, b.cols, a.width)

    def cc_matmul_prepare(self, a, b, target_level=4):
        """First half of singleCCMatMul: sigma(A), tau(B), both at target + 2."""
        sa, tb = self._call("matmul_cc_prepare", a.ct.ptr, *self._shp(a), b.ct.ptr, *self._shp(b), C.c_int(target_level), n_out=2)
        return sa, tb

    def cc_matmul_core(self, sa, tb, rows, inner, cols, width, target_level=4):
        """Second half: the product loop on operands already transformed (any batch)."""
        ct = self._call("matmul_cc_core", sa.ptr, tb.ptr, C.c_int(rows), C.c_int(inner), C.c_int(cols), C.c_int(width), C.c_int(target_level))
        return CtxtTensor(ct, rows, cols, width)

    def packed_matmul(self, a, b, target_level=4):
        ct = self._call("packed_matmul", a.ct.ptr, *self._shp(a), b.ct.ptr, *self._shp(b), C.c_int(target_level))
        return CtxtTensor(ct, a.rows, b.cols, a.width)

    def transpose_inplace(self, t, target_level=0):
        t.ct = self._call("transpose", t.ct.ptr, *self._shp(t), C.c_int(target_level))
        t.rows, t.cols = t.cols, t.rows

    def sigma(self, t):
        return CtxtTensor(self._call("sigma", t.ct.ptr, *self._shp(t)), *t.shape)

    def tau(self, t):
        return CtxtTensor(self._call("tau", t.ct.ptr, *self._shp(t)), *t.shape)

    def matmul_pre(self, a, target_level=4):
        return self._call("matmul_pre", a.ct.ptr, *self._shp(a), C.c_int(target_level))

    def matmul_reuse(self, pre, w):
        return CtxtTensor(self._call("matmul_reuse", pre.ptr, w.ct.ptr, *self._shp(w)), *w.shape)

    def matmul_reuse_groups(self, pre, btotal, b0, weights):
        """Sum over K-groups b0.. of matMulReUse(pre_b, weights[b]); `pre` holds the copies of `btotal` inputs."""
        arr = (C.c_void_p * len(weights))(*[w.ct.ptr.value for w in weights])
        ct = self._call("matmul_reuse_groups", pre.ptr, C.c_int(btotal), C.c_int(b0), arr, C.c_int(len(weights)), C.c_int(weights[0].width))
        return CtxtTensor(ct, *weights[0].shape)

    def matmul_reuse_groups_tiles(self, pre, btotal, b0, weights_by_tile):
        """matmul_reuse_groups for several weight tiles that meet the same copies (all output tiles of a sublayer): one
        pass over the copies per four tiles where the library has the entry point, tile by tile otherwise."""
        f = getattr(self.dll, self.prefix + "matmul_reuse_groups_tiles", None)
        if f is None:
            return [self.matmul_reuse_groups(pre, btotal, b0, ws) for ws in weights_by_tile]
        tiles, bcount = len(weights_by_tile), len(weights_by_tile[0])
        arr = (C.c_void_p * (tiles * bcount))(*[w.ct.ptr.value for ws in weights_by_tile for w in ws])
        outs = (C.c_void_p * tiles)()
        rc = f(self.h, pre.ptr, C.c_int(btotal), C.c_int(b0), arr, C.c_int(bcount), C.c_int(tiles), C.c_int(weights_by_tile[0][0].width), outs)
        if rc != 0:
            g = self._fn("last_error")
            g.restype = C.c_char_p
            raise HBError(rc, g().decode())
        return [CtxtTensor(Handle(self.lib, C.c_void_p(outs[t]), "ct"), *weights_by_tile[0][0].shape) for t in range(tiles)]

    def matmul_pre_rev(self, b, target_level=4):
        return CtxtTensor(self._call("matmul_pre_rev", b.ct.ptr, *self._shp(b), C.c_int(target_level)), *b.shape)

    def matmul_cc_reuse(self, pre, b):
        return CtxtTensor(self._call("matmul_cc_reuse", pre.ptr, b.ct.ptr, *self._shp(b)), *b.shape)

    def packed_matmul_pre(self, a, target_level=4):
        return CtxtTensor(self._call("packed_matmul_pre", a.ct.ptr, *self._shp(a), C.c_int(target_level)), *a.shape)

    def packed_matmul_pre_rot(self, a, target_level=4):
        return self._call("packed_matmul_pre_rot", a.ct.ptr, *self._shp(a), C.c_int(target_level))

    def packed_matmul_pre_rev(self, b, target_level=4):
        return CtxtTensor(self._call("packed_matmul_pre_rev", b.ct.ptr, *self._shp(b), C.c_int(target_level)), *b.shape)

    def packed_matmul_cc_reuse(self, pre, b):
        return CtxtTensor(self._call("packed_matmul_cc_reuse", pre.ptr, b.ct.ptr, *self._shp(b)), *b.shape)

    # ---- packing helpers ----
    def complex_packing_inplace(self, t):
        t.ct = self._call("complex_packing", t.ct.ptr, *self._shp(t))

    def complex_packing_row_inplace(self, t):
        t.ct = self._call("complex_packing_row", t.ct.ptr, *self._shp(t))

    def transpose_complex_packing_inplace(self, t, target_level=0):
        t.ct = self._call("transpose_complex_packing", t.ct.ptr, *self._shp(t), C.c_int(target_level))
        t.rows, t.cols = t.cols, t.rows

    def split_in_two(self, t):
        a, b = self._call("split_in_two", t.ct.ptr, *self._shp(t), n_out=2)
        return CtxtTensor(a, *t.shape), CtxtTensor(b, *t.shape)

    def repack_cc(self, t):
        return CtxtTensor(self._call("repack_cc", t.ct.ptr), *t.shape)

    def complex_packing(self, a, b):
        return CtxtTensor(self._call("complex_packing2", a.ct.ptr, b.ct.ptr), *b.shape)

    def complex_packing_rev(self, a, b):
        return CtxtTensor(self._call("complex_packing_rev", a.ct.ptr, b.ct.ptr), *b.shape)

    def repack_not_bts(self, a, b):
        return CtxtTensor(self._call("repack_not_bts", a.ct.ptr, b.ct.ptr), *a.shape)

    def repack_lora_opti(self, a, b):
        return CtxtTensor(self._call("repack_lora_opti", a.ct.ptr, b.ct.ptr), *a.shape)

    # ---- LoRA low-rank products (HEMMer.hpp:326-346) ----
    def matmul_high_low(self, a, b, in_col_block, target_level=4, low_dim=2):
        """HEMMer::matMulHighLow: full tile x thin block that sits in column block `in_col_block`."""
        ct = self._call("matmul_high_low", a.ct.ptr, *self._shp(a), b.ct.ptr, *self._shp(b),
                        C.c_int(in_col_block), C.c_int(target_level), C.c_int(low_dim))
        return CtxtTensor(ct, a.rows, b.cols, b.width)

    def matmul_low_high(self, a, b, in_row_block, target_level=4, low_dim=2):
        """HEMMer::matMulLowHigh: thin block in row block `in_row_block` x full tile."""
        ct = self._call("matmul_low_high", a.ct.ptr, *self._shp(a), b.ct.ptr, *self._shp(b),
                        C.c_int(in_row_block), C.c_int(target_level), C.c_int(low_dim))
        return CtxtTensor(ct, a.rows, b.cols, b.width)

    def matmul_low_low(self, a, b, in_col_block, in_row_block, target_level=4, low_dim=2):
        """HEMMer::matMulLowLow: thin column block x thin row block."""
        ct = self._call("matmul_low_low", a.ct.ptr, *self._shp(a), b.ct.ptr, *self._shp(b),
                        C.c_int(in_col_block), C.c_int(in_row_block), C.c_int(target_level), C.c_int(low_dim))
        return CtxtTensor(ct, a.rows, b.cols, b.width)

    def _low(self, name, t, block, low_dim):
        return CtxtTensor(self._call(name, t.ct.ptr, *self._shp(t), C.c_int(block), C.c_int(low_dim)), *t.shape)

    def repack_to_one_col(self, t, out_col_block, low_dim=2):
        return self._low("repack_to_one_col", t, out_col_block, low_dim)

    def repack_to_multi_col(self, t, out_col_block, low_dim=2):
        return self._low("repack_to_multi_col", t, out_col_block, low_dim)

    def repack_to_one_row(self, t, out_row_block, low_dim=2):
        return self._low("repack_to_one_row", t, out_row_block, low_dim)

    def repack_to_multi_row(self, t, out_row_block, low_dim=2):
        return self._low("repack_to_multi_row", t, out_row_block, low_dim)

    def get_low_col_block(self, t, col_block, low_dim=2):
        return self._low("low_col_block", t, col_block, low_dim)

    def get_low_row_block(self, t, row_block, low_dim=2):
        return self._low("low_row_block", t, row_block, low_dim)
