"""ctypes binding of the C ABI declared in include/hemmer_b200.h.

The same binding class drives any shared library that exports that ABI under a
symbol prefix; the shipped CUDA library uses the prefix ``hb_``.  Nothing in this
module computes anything: every call lands in native code.
"""
from __future__ import annotations

import ctypes as C
import numpy as np

c_u64p = C.POINTER(C.c_uint64)
c_f64p = C.POINTER(C.c_double)
c_i64p = C.POINTER(C.c_int64)


class Params(C.Structure):
    """Mirror of ``hb_params``."""

    _fields_ = [
        ("log_n", C.c_int32), ("max_level", C.c_int32), ("dnum", C.c_int32), ("num_special", C.c_int32),
        ("q0_bits", C.c_int32), ("q_bits", C.c_int32), ("p_bits", C.c_int32), ("hamming_weight", C.c_int32),
        ("sigma", C.c_double), ("seed", C.c_uint64 * 4),
    ]


def make_params(log_n=16, max_level=12, dnum=4, num_special=3, q0_bits=60, q_bits=42, p_bits=60,
                hamming_weight=192, sigma=3.2, seed=(0x243F6A8885A308D3, 0x13198A2E03707344,
                                                     0xA4093822299F31D0, 0x082EFA98EC4E6C89)) -> Params:
    p = Params(log_n, max_level, dnum, num_special, q0_bits, q_bits, p_bits, hamming_weight, sigma)
    for i in range(4):
        p.seed[i] = seed[i]
    return p


class HBError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"[{code}] {msg}")
        self.code = code


def _f64(a):
    return None if a is None else a.ctypes.data_as(c_f64p)


class Handle:
    """A ciphertext-batch or plaintext handle owned by Python."""

    def __init__(self, lib, ptr, kind):
        self.lib, self.ptr, self.kind = lib, ptr, kind

    def __del__(self):
        if getattr(self, "ptr", None) and self.lib is not None and self.lib.alive:
            f = getattr(self.lib.dll, f"{self.lib.prefix}{self.kind}_free")
            f.restype = None
            f(self.ptr)
            self.ptr = None


class Lib:
    """One loaded library + one context."""

    def __init__(self, path: str, prefix: str, params: Params, device: int = 0):
        self.dll = C.CDLL(path)
        self.prefix = prefix
        self.alive = False
        self.params = params
        f = self._fn
        self.ctx = C.c_void_p()
        rc = f("ctx_create")(C.byref(params), C.c_int(device), C.byref(self.ctx))
        if rc != 0:
            raise HBError(rc, "ctx_create failed (no CUDA device or bad parameters)")
        self.alive = True
        f("last_error").restype = C.c_char_p
        f("galois_for_rotation").restype = C.c_uint64
        for name in ("ct_free", "pt_free", "ctx_destroy"):
            f(name).restype = None
        self.N = 1 << params.log_n
        self.slots = self.N // 2
        self.L = params.max_level
        self.K = params.num_special
        pr = np.zeros(self.L + 1 + self.K, dtype=np.uint64)
        sc = np.zeros(self.L + 1, dtype=np.float64)
        self._chk(f("ctx_info")(self.ctx, pr.ctypes.data_as(c_u64p), _f64(sc)))
        self.primes, self.scales = pr, sc

    def _fn(self, name):
        return getattr(self.dll, self.prefix + name)

    def has(self, name):
        return hasattr(self.dll, self.prefix + name)

    def _chk(self, rc):
        if rc != 0:
            raise HBError(rc, self._fn("last_error")(self.ctx).decode())

    def close(self):
        if self.alive:
            self.alive = False
            self._fn("ctx_destroy")(self.ctx)

    # ---- keys ----
    def keygen(self):
        self._chk(self._fn("keygen")(self.ctx))

    def gen_rot_keys(self, steps):
        a = np.asarray(list(steps), dtype=np.int64)
        self._chk(self._fn("gen_rot_keys")(self.ctx, a.ctypes.data_as(c_i64p), C.c_int(len(a))))

    def galois(self, steps):
        return int(self._fn("galois_for_rotation")(self.ctx, C.c_int64(steps)))

    def evk_export(self, galois):
        nd = C.c_int(0)
        self._chk(self._fn("evk_export")(self.ctx, C.c_uint64(galois), None, C.byref(nd)))
        out = np.zeros((nd.value, 2, self.L + 1 + self.K, self.N), dtype=np.uint64)
        self._chk(self._fn("evk_export")(self.ctx, C.c_uint64(galois), out.ctypes.data_as(c_u64p), C.byref(nd)))
        return out

    # ---- encode / encrypt ----
    def encode(self, z, level):
        z = np.asarray(z)
        re = np.ascontiguousarray(z.real, dtype=np.float64)
        im = np.ascontiguousarray(z.imag, dtype=np.float64) if np.iscomplexobj(z) else None
        out = C.c_void_p()
        self._chk(self._fn("encode")(self.ctx, _f64(re), _f64(im), C.c_size_t(re.size), C.c_int(level), C.byref(out)))
        return Handle(self, out, "pt")

    def encode_ext(self, z, level):
        """encode() with K further limbs modulo the special primes: the plaintext operand of assemble_rot."""
        z = np.asarray(z)
        re = np.ascontiguousarray(z.real, dtype=np.float64)
        im = np.ascontiguousarray(z.imag, dtype=np.float64) if np.iscomplexobj(z) else None
        out = C.c_void_p()
        self._chk(self._fn("encode_ext")(self.ctx, _f64(re), _f64(im), C.c_size_t(re.size), C.c_int(level), C.byref(out)))
        return Handle(self, out, "pt")

    def decode(self, pt):
        re = np.zeros(self.slots); im = np.zeros(self.slots)
        self._chk(self._fn("decode")(self.ctx, pt.ptr, _f64(re), _f64(im)))
        return re + 1j * im

    def encrypt(self, pt, nonce):
        out = C.c_void_p()
        self._chk(self._fn("encrypt")(self.ctx, pt.ptr, C.c_uint64(nonce), C.byref(out)))
        return Handle(self, out, "ct")

    def decrypt(self, ct, index=0):
        re = np.zeros(self.slots); im = np.zeros(self.slots)
        self._chk(self._fn("decrypt")(self.ctx, ct.ptr, C.c_int(index), _f64(re), _f64(im)))
        return re + 1j * im

    def encrypt_many(self, msgs, level, nonces):
        """Encode + encrypt the rows of `msgs` ([count][slots], real or complex) into one batched handle."""
        msgs = np.asarray(msgs)
        n = msgs.shape[0]
        if not self.has("encrypt_many"):  # a library without the batched entry point: one call per member
            return self.batch_concat([self.encrypt(self.encode(m, level), k) for m, k in zip(msgs, nonces)])
        re = np.ascontiguousarray(msgs.real, dtype=np.float64)
        im = np.ascontiguousarray(msgs.imag, dtype=np.float64) if np.iscomplexobj(msgs) else None
        nn = (C.c_uint64 * n)(*[int(k) for k in nonces])
        out = C.c_void_p()
        self._chk(self._fn("encrypt_many")(self.ctx, _f64(re), _f64(im), C.c_size_t(msgs.shape[1]), C.c_int(n), C.c_int(level), nn, C.byref(out)))
        return Handle(self, out, "ct")

    def decrypt_many(self, items):
        """Decrypt a list of (ciphertext handle, batch index) pairs in one call; returns complex [len(items)][slots]."""
        n = len(items)
        if not self.has("decrypt_many"):  # a library without the batched entry point: one call per member
            return np.stack([self.decrypt(ct, k) for ct, k in items])
        re = np.zeros((n, self.slots)); im = np.zeros((n, self.slots))
        cts = (C.c_void_p * n)(*[ct.ptr.value for ct, _ in items])
        idx = (C.c_int * n)(*[int(k) for _, k in items])
        self._chk(self._fn("decrypt_many")(self.ctx, cts, idx, C.c_int(n), _f64(re), _f64(im)))
        return re + 1j * im

    # ---- raw ----
    def ct_create(self, level, n_poly=2, batch=1, scale_pow=1):
        out = C.c_void_p()
        self._chk(self._fn("ct_create")(self.ctx, C.c_int(level), C.c_int(n_poly), C.c_int(batch), C.c_int(scale_pow), C.byref(out)))
        return Handle(self, out, "ct")

    def ct_meta(self, ct):
        v = [C.c_int() for _ in range(4)]
        self._fn("ct_meta")(ct.ptr, *[C.byref(x) for x in v])
        return tuple(x.value for x in v)  # level, n_poly, batch, scale_pow

    def pt_meta(self, pt):
        v = [C.c_int() for _ in range(2)]
        self._fn("pt_meta")(pt.ptr, *[C.byref(x) for x in v])
        return tuple(x.value for x in v)

    def ct_import(self, ct, arr):
        arr = np.ascontiguousarray(arr, dtype=np.uint64)
        self._chk(self._fn("ct_import")(self.ctx, ct.ptr, arr.ctypes.data_as(c_u64p)))

    def ct_export(self, ct):
        level, npoly, batch, _ = self.ct_meta(ct)
        out = np.zeros((batch, npoly, level + 1, self.N), dtype=np.uint64)
        self._chk(self._fn("ct_export")(self.ctx, ct.ptr, out.ctypes.data_as(c_u64p)))
        return out

    def pt_export(self, pt):
        level, _ = self.pt_meta(pt)
        out = np.zeros((level + 1, self.N), dtype=np.uint64)
        self._chk(self._fn("pt_export")(self.ctx, pt.ptr, out.ctypes.data_as(c_u64p)))
        return out

    # ---- files (the library's own container; see include/hemmer_b200.h) ----
    def ct_save(self, ct, path):
        self._chk(self._fn("ct_save")(self.ctx, ct.ptr, str(path).encode()))

    def ct_load(self, path):
        out = C.c_void_p()
        self._chk(self._fn("ct_load")(self.ctx, str(path).encode(), C.byref(out)))
        return Handle(self, out, "ct")

    def pt_save(self, pt, path):
        self._chk(self._fn("pt_save")(self.ctx, pt.ptr, str(path).encode()))

    def pt_load(self, path):
        out = C.c_void_p()
        self._chk(self._fn("pt_load")(self.ctx, str(path).encode(), C.byref(out)))
        return Handle(self, out, "pt")

    def keys_save(self, directory):
        self._chk(self._fn("keys_save")(self.ctx, str(directory).encode()))

    def keys_load(self, directory, galois=()):
        g = (C.c_uint64 * max(1, len(galois)))(*[int(x) for x in galois])
        self._chk(self._fn("keys_load")(self.ctx, str(directory).encode(), g, C.c_int(len(galois))))

    def batch_set(self, dst, idx, src):
        self._chk(self._fn("batch_set")(self.ctx, dst.ptr, C.c_int(idx), src.ptr))

    def batch_get(self, src, idx):
        out = C.c_void_p()
        self._chk(self._fn("batch_get")(self.ctx, src.ptr, C.c_int(idx), C.byref(out)))
        return Handle(self, out, "ct")

    def ct_zero(self, ct):
        self._chk(self._fn("ct_zero")(self.ctx, ct.ptr))

    def allreduce_sum(self, ct, comm):
        """Sum over the ranks of `comm` (an NCCL communicator as an integer address), then reduce modulo each prime."""
        self._chk(self._fn("allreduce_sum")(self.ctx, ct.ptr, C.c_void_p(comm)))

    def reduce_sum(self, ct, root, my_rank, comm):
        """Sum over the ranks to `root`, which then reduces modulo each prime; other ranks keep their buffer."""
        self._chk(self._fn("reduce_sum")(self.ctx, ct.ptr, C.c_int(root), C.c_int(my_rank), C.c_void_p(comm)))

    def allgather(self, mine, all_, comm):
        """`all_` (batch = ranks x batch of `mine`) receives every rank's `mine`, rank-major."""
        self._chk(self._fn("allgather")(self.ctx, mine.ptr, all_.ptr, C.c_void_p(comm)))

    def nccl_group_start(self):
        rc = self._fn("nccl_group_start")()
        if rc != 0:
            raise HBError(rc, "ncclGroupStart failed")

    def nccl_group_end(self):
        rc = self._fn("nccl_group_end")()
        if rc != 0:
            raise HBError(rc, "ncclGroupEnd failed")

    def send(self, ct, peer, comm):
        self._chk(self._fn("send")(self.ctx, ct.ptr, C.c_int(peer), C.c_void_p(comm)))

    def recv(self, ct, peer, comm):
        self._chk(self._fn("recv")(self.ctx, ct.ptr, C.c_int(peer), C.c_void_p(comm)))

    def sum_mod_reduce(self, parts):
        """(sum of the parts) mod q in one pass: the owner's half of a K-split exchange."""
        arr = (C.c_void_p * len(parts))(*[p.ptr.value for p in parts])
        return self._op("sum_mod_reduce", arr, C.c_int(len(parts)))

    def mod_reduce(self, ct):
        self._chk(self._fn("mod_reduce")(self.ctx, ct.ptr))

    def set_host_threads(self, n):
        self._chk(self._fn("set_host_threads")(self.ctx, C.c_int(n)))

    # ---- CUDA graph of a fixed call sequence ----
    def graph_begin(self):
        self._chk(self._fn("graph_begin")(self.ctx))

    def graph_end(self):
        out = C.c_void_p()
        self._chk(self._fn("graph_end")(self.ctx, C.byref(out)))
        return Handle(self, out, "graph")

    def graph_launch(self, g):
        self._chk(self._fn("graph_launch")(self.ctx, g.ptr))

    def graph_kernels(self, g):
        f = self._fn("graph_kernels")
        f.restype = C.c_uint64
        return int(f(g.ptr))

    def batch_concat(self, parts):
        arr = (C.c_void_p * len(parts))(*[p.ptr.value for p in parts])
        out = C.c_void_p()
        self._chk(self._fn("batch_concat")(self.ctx, arr, C.c_int(len(parts)), C.byref(out)))
        return Handle(self, out, "ct")

    def batch_slice(self, src, start, count):
        out = C.c_void_p()
        self._chk(self._fn("batch_slice")(self.ctx, src.ptr, C.c_int(start), C.c_int(count), C.byref(out)))
        return Handle(self, out, "ct")

    def sync(self):
        self._chk(self._fn("sync")(self.ctx))

    # ---- primitives ----
    def _op(self, name, *args):
        out = C.c_void_p()
        self._chk(self._fn(name)(self.ctx, *args, C.byref(out)))
        return Handle(self, out, "ct")

    def add(self, a, b): return self._op("add", a.ptr, b.ptr)
    def sub(self, a, b): return self._op("sub", a.ptr, b.ptr)
    def negate(self, a): return self._op("negate", a.ptr)
    def mult_imag(self, a): return self._op("mult_imag", a.ptr)
    def mult_int(self, a, k): return self._op("mult_int", a.ptr, C.c_int64(k))
    def mul_pt(self, a, p): return self._op("mul_pt", a.ptr, p.ptr)
    def mul_pt_norescale(self, a, p): return self._op("mul_pt_norescale", a.ptr, p.ptr)
    def rescale(self, a): return self._op("rescale", a.ptr)
    def level_down(self, a, t): return self._op("level_down", a.ptr, C.c_int(t))
    def tensor(self, a, b): return self._op("tensor", a.ptr, b.ptr)
    def relin(self, a): return self._op("relin", a.ptr)
    def mul(self, a, b): return self._op("mul", a.ptr, b.ptr)
    def rotate(self, a, s): return self._op("rotate", a.ptr, C.c_int64(s))
    def conjugate(self, a): return self._op("conjugate", a.ptr)

    def rotate_sum(self, xs, steps):
        """sum_t rot(xs[t], steps[t]) with one ModDown for the whole sum."""
        n = len(xs)
        arr = (C.c_void_p * n)(*[x.ptr.value for x in xs])
        st = (C.c_int64 * n)(*[int(v) for v in steps])
        return self._op("rotate_sum", arr, st, C.c_int(n))

    def assemble_rot(self, a, s1, p1, s2, p2):
        """rescale(p1 (.) rot(a, s1) + p2 (.) rot(a, s2)) with one division by P * q_level for the sum."""
        return self._op("assemble_rot", a.ptr, C.c_int64(s1), p1.ptr, C.c_int64(s2), p2.ptr)

    # ---- hoisting (CUDA library only: the oracle defines rotation as decompose-then-permute and has no split) ----
    def decompose(self, a):
        out = C.c_void_p()
        self._chk(self._fn("decompose")(self.ctx, a.ptr, C.byref(out)))
        return Handle(self, out, "digits")

    def rotate_hoisted(self, a, digits, s): return self._op("rotate_hoisted", a.ptr, digits.ptr, C.c_int64(s))

    def masked_key(self, steps, m1, m2=None):
        """Rotation key of `steps` multiplied by the extended plaintext m1 (+ m2), for the plaintexts' level."""
        out = C.c_void_p()
        self._chk(self._fn("masked_key_create")(self.ctx, C.c_int64(steps), m1.ptr, m2.ptr if m2 is not None else None, C.byref(out)))
        return Handle(self, out, "masked_key")

    def assemble_masked(self, a, digits, k1, k2=None):
        return self._op("assemble_masked", a.ptr, digits.ptr, k1.ptr, k2.ptr if k2 is not None else None)

    def _pt_op(self, name, *args):
        out = C.c_void_p()
        self._chk(self._fn(name)(self.ctx, *args, C.byref(out)))
        return Handle(self, out, "pt")

    def pt_mul(self, a, b): return self._pt_op("pt_mul", a.ptr, b.ptr)
    def pt_add(self, a, b): return self._pt_op("pt_add", a.ptr, b.ptr)
    def pt_rotate(self, a, s): return self._pt_op("pt_rotate", a.ptr, C.c_int64(s))

    def ntt(self, a, inverse=False):
        self._chk(self._fn("ntt")(self.ctx, a.ptr, C.c_int(1 if inverse else 0)))
