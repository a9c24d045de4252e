"""BERT-base encoder-layer matmul workload over HEMMer (forward + LoRA backward), tile-sharded.

Shapes follow the reference's micro-benchmarks (ciphertext/examples/bert-matmul.cpp,
bert-matmul-backward.cpp): 128 tokens, hidden 768 = 6 tiles of 128, FFN 3072 = 24 tiles, two tiles per
ciphertext ([A | B], HEMMer::encrypt2), plaintext weights packed four tiles per plaintext
(HEMMer::encodeDiagonalToRow4).  As in those programs every matmul starts from freshly encrypted
top-level operands; the non-linear steps between them (softmax, layer norm, bootstrapping) are not
part of the workload.

Work items are independent "units" (one matMulPre group with its matMulReUse products, or one
two-tile ct x ct product); rank r of R executes units r, r+R, ... so the same code runs on 1..8 GPUs.
"""
from __future__ import annotations

import numpy as np

from .hemmer import CtxtTensor, Hemmer

D = 128          # tile side
HIDDEN = 6       # 768 / 128
FFN = 24         # 3072 / 128
HEADS = 12
LORA_RANK = 8


def synthetic(seed: int):
    """Seeded inputs with BASELINE's distributions: activations U[-1,1], weights N(0, 0.02^2)."""
    rng = np.random.default_rng(seed)
    u = lambda *s: rng.uniform(-1.0, 1.0, s)
    w = lambda *s: rng.normal(0.0, 0.02, s)
    data = {
        "x": u(D, 768), "wq": w(768, 768), "wk": w(768, 768), "wv": w(768, 768), "wo": w(768, 768),
        "w1": w(768, 3072), "w2": w(3072, 768), "h": u(D, 3072),
        "q": u(HEADS, D, 64), "k": u(HEADS, D, 64), "v": u(HEADS, D, 64), "s": rng.uniform(0.0, 1.0 / 128, (HEADS, D, D)),
        "lora_a": [w(768, LORA_RANK) for _ in range(2)], "lora_b": [w(LORA_RANK, 768) for _ in range(2)],
        "dy": [u(D, 768) for _ in range(2)],
    }
    return data


def tiles(m, r, c):
    """Tile (r, c) of a matrix, zero-padded to D x D."""
    blk = m[r * D:(r + 1) * D, c * D:(c + 1) * D]
    out = np.zeros((D, D))
    out[: blk.shape[0], : blk.shape[1]] = blk
    return out


class LayerWorkload:
    """Builds the unit list once (weights encoded, masks and keys warmed by the first step)."""

    def __init__(self, H: Hemmer, data, rank: int = 0, world: int = 1, target: int = 4):
        self.H, self.lib, self.data, self.rank, self.world, self.target = H, H.lib, data, rank, world, target
        self.units = self._build_units()
        self.mine = [u for i, u in enumerate(self.units) if i % world == rank]
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self._weights = {}

    # ---- unit construction ----
    def _build_units(self):
        d = self.data
        units = []
        # ct x pt: one unit per group of four K-tiles (matMulPre) with all its output tiles (matMulReUse)
        def pcmm(name, x, weights, kt, nt):
            for g in range((kt + 3) // 4):
                units.append(("pcmm", name, x, weights, g, kt, nt))
        pcmm("qkv", "x", ["wq", "wk", "wv"], HIDDEN, HIDDEN)
        pcmm("wo", "x", ["wo"], HIDDEN, HIDDEN)
        pcmm("w1", "x", ["w1"], HIDDEN, FFN)
        pcmm("w2", "h", ["w2"], FFN, HIDDEN)
        # ct x ct, two tiles per ciphertext
        for ad in range(2):                      # LoRA forward: X*A (K-split over 3 pairs) and (XA)*B (3 output pairs)
            for p in range(3):
                units.append(("ccmm", f"lora{ad}_xa{p}", ("x_pair", p), ("a_pair", ad, p), False))
            for p in range(3):
                units.append(("ccmm", f"lora{ad}_xab{p}", ("xa_rep", ad), ("b_pair", ad, p), False))
        for hp in range(HEADS // 2):             # attention: Q*K^T and S*V, two heads per ciphertext
            units.append(("ccmm", f"qk{hp}", ("head", "q", hp), ("head", "k", hp), True))
            units.append(("ccmm", f"sv{hp}", ("score", hp), ("head", "v", hp), False))
        for ad in range(2):                      # LoRA backward: dB = (XA)^T dY, d(XA) = dY B^T, dA = X^T d(XA)
            for p in range(3):
                units.append(("ccmm", f"bwd{ad}_db{p}", ("xa_rep", ad), ("dy_pair", ad, p), "left"))
                units.append(("ccmm", f"bwd{ad}_dxa{p}", ("dy_pair", ad, p), ("b_pair", ad, p), True))
                units.append(("ccmm", f"bwd{ad}_da{p}", ("x_pair", p), ("dxa_rep", ad), "left"))
        return units

    # ---- operand materialisation (host matrices -> tiles) ----
    def _pair(self, spec):
        d = self.data
        kind = spec[0]
        if kind == "x_pair":
            return tiles(d["x"], 0, 2 * spec[1]), tiles(d["x"], 0, 2 * spec[1] + 1)
        if kind == "a_pair":
            a = d["lora_a"][spec[1]]
            return tiles(a, 2 * spec[2], 0), tiles(a, 2 * spec[2] + 1, 0)
        if kind == "b_pair":
            b = d["lora_b"][spec[1]]
            return tiles(b, 0, 2 * spec[2]), tiles(b, 0, 2 * spec[2] + 1)
        if kind == "xa_rep":
            xa = tiles(d["x"] @ d["lora_a"][spec[1]], 0, 0)
            return xa, xa
        if kind == "dxa_rep":
            dxa = tiles(d["dy"][spec[1]] @ d["lora_b"][spec[1]].T, 0, 0)
            return dxa, dxa
        if kind == "dy_pair":
            dy = d["dy"][spec[1]]
            return tiles(dy, 0, 2 * spec[2]), tiles(dy, 0, 2 * spec[2] + 1)
        if kind == "head":
            m = d[spec[1]]
            pad = lambda h: np.pad(m[h], ((0, 0), (0, D - 64)))
            return pad(2 * spec[2]), pad(2 * spec[2] + 1)
        if kind == "score":
            return d["s"][2 * spec[1]], d["s"][2 * spec[1] + 1]
        raise KeyError(kind)

    def _encrypt_pair(self, spec, nonce):
        a, b = self._pair(spec)
        self.h2d_bytes += 2 * self.lib.N * 8
        return self.H.encrypt2(a, b, nonce=nonce), (a, b)

    def _weight_pts(self, wname, g, kt, nt):
        key = (wname, g)
        if key not in self._weights:
            w = self.data[wname]
            z = np.zeros((D, D))
            pts = []
            for j in range(nt):
                t = [tiles(w, 4 * g + i, j) if 4 * g + i < kt else z for i in range(4)]
                pts.append(self.H.encode_diagonal_to_row4(*t, level=self.target + 1))
            self._weights[key] = pts
        return self._weights[key]

    # ---- execution ----
    def _operands(self, u, nonce0):
        """Encode + encrypt the unit's operands from host matrices (host -> device traffic)."""
        H, lib = self.H, self.lib
        per_ct = 2 * lib.N * 8  # rounded message coefficients + error polynomial uploaded per encryption
        if u[0] == "pcmm":
            _, name, xname, weights, g, kt, nt = u
            x = self.data[xname]
            pair = lambda p: (tiles(x, 0, 2 * p), tiles(x, 0, 2 * p + 1))
            cts = [H.encrypt2(*pair(2 * g), nonce=nonce0)]
            if 4 * g + 2 < kt:
                cts.append(H.encrypt2(*pair(2 * g + 1), nonce=nonce0 + 1))
            self.h2d_bytes += per_ct * len(cts)
            for wname in weights:
                self._weight_pts(wname, g, kt, nt)
            return cts
        _, name, lhs, rhs, tr = u
        a, b = self._pair(lhs), self._pair(rhs)
        self.h2d_bytes += 2 * per_ct
        return [H.encrypt2(*a, nonce=nonce0), H.encrypt2(*b, nonce=nonce0 + 1)]

    def _compute(self, u, cts):
        H, t = self.H, self.target
        if u[0] == "pcmm":
            _, name, xname, weights, g, kt, nt = u
            packed = H.complex_packing(cts[0], cts[1]) if len(cts) == 2 else cts[0]
            pre = H.matmul_pre(packed, t)
            return [H.matmul_reuse(pre, pt) for wname in weights for pt in self._weight_pts(wname, g, kt, nt)]
        _, name, lhs, rhs, tr = u
        a = CtxtTensor(cts[0].ct, *cts[0].shape)
        b = CtxtTensor(cts[1].ct, *cts[1].shape)
        if tr is True:
            H.transpose_inplace(b)
        elif tr == "left":
            H.transpose_inplace(a)
        return [H.single_cc_matmul(a, b, t)]

    def _expected(self, u):
        if u[0] == "pcmm":
            _, name, xname, weights, g, kt, nt = u
            x, w = self.data[xname], self.data[weights[0]]
            return sum(tiles(x, 0, 4 * g + i) @ tiles(w, 4 * g + i, 0) for i in range(4) if 4 * g + i < kt)
        _, name, lhs, rhs, tr = u
        (a0, a1), (b0, b1) = self._pair(lhs), self._pair(rhs)
        if tr is True:
            b0, b1 = b0.T, b1.T
        elif tr == "left":
            a0, a1 = a0.T, a1.T
        return np.stack([a0 @ b0, a1 @ b1])

    def _decrypted(self, u, out):
        """Device -> host: decrypt the first result of the unit into matrices."""
        self.d2h_bytes += 2 * self.lib.N * 8
        if u[0] == "pcmm":
            z = self.lib.decrypt(out[0].ct).reshape(D, 2 * D)
            return 2 * (z[:, :D].real + z[:, D:].real)
        return self.H.decrypt2(out[0])

    def prepare(self):
        """Make every operand of this rank's units resident on the device."""
        self.resident = [self._operands(u, 10_000 + 16 * i) for i, u in enumerate(self.mine)]

    def step_resident(self):
        last = None
        for u, cts in zip(self.mine, self.resident):
            last = self._compute(u, cts)
        return last

    def step(self):
        last = None
        for i, u in enumerate(self.mine):
            last = self._compute(u, self._operands(u, 10_000 + 16 * i))
        return last

    def step_e2e(self):
        """Host matrices in, decrypted host matrices out, for every unit."""
        res = None
        for i, u in enumerate(self.mine):
            out = self._compute(u, self._operands(u, 30_000 + 16 * i))
            res = self._decrypted(u, out)
        return res

    def check(self, which=(0, -1)):
        """Max-abs error of a few units against the float64 products."""
        err = 0.0
        for k in which:
            if not self.mine:
                break
            u = self.mine[k]
            out = self._compute(u, self._operands(u, 20_000 + 16 * (k % 1000)))
            err = max(err, float(np.abs(self._decrypted(u, out) - self._expected(u)).max()))
        return err
