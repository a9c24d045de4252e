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

import time

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
    """The layer's matmuls as a few large batched calls.

    ct x pt: the K-groups of all four sublayers go through complexPacking + matMulPre as one batch
    (groups with two ciphertexts and groups with one are separate batches, because they are packed
    differently); every output tile is then one fused pass over the shifted copies of its sublayer's
    groups.  ct x ct: the 42 products share one schedule, so they run as three batches (no transpose,
    right operand transposed, left operand transposed).  Every batch entry is computed exactly as it
    would be alone; batching only puts more ciphertexts behind each kernel launch.
    """

    PCMM = [("qkv", "x", ["wq", "wk", "wv"], HIDDEN, HIDDEN), ("wo", "x", ["wo"], HIDDEN, HIDDEN),
            ("w1", "x", ["w1"], HIDDEN, FFN), ("w2", "h", ["w2"], FFN, HIDDEN)]

    def __init__(self, H: Hemmer, data, rank: int = 0, world: int = 1, target: int = 4):
        self.H, self.lib, self.data, self.rank, self.world, self.target = H, H.lib, data, rank, world, target
        self.units = self._build_units()
        self.mine = [u for i, u in enumerate(self.units) if i % world == rank]
        self.h2d_bytes = 0
        self.phases_ms = {}
        self.d2h_bytes = 0
        self._weights = {}
        self.resident = None
        self.comm = None   # NCCL communicator (void*) when several ranks split the K-groups of a sublayer

    # ---- unit construction ----
    def _build_units(self):
        units = []
        for name, x, weights, kt, nt in self.PCMM:
            for g in range((kt + 3) // 4):
                units.append(("pcmm", name, x, weights, g, kt, nt))
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

    def _batch(self, cts):
        """Gather single ciphertexts into one batched handle (device-to-device copies)."""
        lib = self.lib
        level, npoly, _, spow = lib.ct_meta(cts[0].ct)
        out = lib.ct_create(level, npoly, len(cts), spow)
        for k, c in enumerate(cts):
            lib.batch_set(out, k, c.ct)
        return CtxtTensor(out, *cts[0].shape)

    # ---- host -> device ----
    def _encrypt_all(self, nonce0):
        """Encode + encrypt every operand of this rank's units, one batched call per group of operands."""
        H, lib = self.H, self.lib
        per_ct = 2 * lib.N * 8  # rounded message coefficients + error polynomial uploaded per encryption
        groups = {"full": [], "half": []}      # pcmm: (unit, [(pair, nonce)])
        ccmm = {False: [], True: [], "left": []}
        n = nonce0
        for u in self.mine:
            if u[0] == "pcmm":
                _, name, xname, weights, g, kt, nt = u
                x = self.data[xname]
                pair = lambda p: (tiles(x, 0, 2 * p), tiles(x, 0, 2 * p + 1))
                ops = [(pair(2 * g), n)]
                if 4 * g + 2 < kt:
                    ops.append((pair(2 * g + 1), n + 1))
                self.h2d_bytes += per_ct * len(ops)
                for wname in weights:
                    self._weight_pts(wname, g, kt, nt)
                groups["full" if len(ops) == 2 else "half"].append((u, ops))
            else:
                _, name, lhs, rhs, tr = u
                self.h2d_bytes += 2 * per_ct
                ccmm[tr].append((u, (self._pair(lhs), n), (self._pair(rhs), n + 1)))
            n += 2
        many = lambda ops: H.encrypt2_many([p for p, _ in ops], [k for _, k in ops])
        res = {"pcmm": {}, "ccmm": {}}
        for kind, lst in groups.items():
            if lst:
                res["pcmm"][kind] = ([u for u, _ in lst], many([o[0] for _, o in lst]),
                                     many([o[1] for _, o in lst]) if kind == "full" else None)
        for tr, lst in ccmm.items():
            if lst:
                res["ccmm"][tr] = ([u for u, _, _ in lst], many([a for _, a, _ in lst]), many([b for _, _, b in lst]))
        return res

    # ---- device work ----
    def _compute(self, res):
        H, t = self.H, self.target
        out = {"pcmm": {}, "ccmm": {}}
        pres = {}
        for kind, (us, c01, c23) in res["pcmm"].items():
            packed = H.complex_packing(c01, c23) if c23 is not None else c01
            pres[kind] = (us, H.matmul_pre(packed, t))
        # every (sublayer, weight, output tile): one fused pass per batch of K-groups, partial sums added
        for name, xname, weights, kt, nt in self.PCMM:
            for wname in weights:
                for j in range(nt):
                    acc = None
                    for kind, (us, pre) in pres.items():
                        sel = [(b, u) for b, u in enumerate(us) if u[1] == name]
                        if not sel:
                            continue
                        b0 = sel[0][0]
                        pts = [self._weight_pts(wname, u[4], kt, nt)[j] for _, u in sel]
                        part = H.matmul_reuse_groups(pre, len(us), b0, pts)
                        acc = part if acc is None else CtxtTensor(self.lib.add(acc.ct, part.ct), *part.shape)
                    if acc is not None:
                        out["pcmm"][(name, wname, j)] = acc
        if self.world > 1:
            self._reduce_partials(out["pcmm"])
        # ct x ct: one batched transpose for every operand that needs it; the transforms sigma / tau run per group
        # (a transposed tile sits one level lower), then ONE product loop serves all units of this rank
        cc = res["ccmm"]
        if cc:
            lib = self.lib
            order = [tr for tr in (False, True, "left") if tr in cc]
            need = [cc[tr][2] if tr is True else cc[tr][1] for tr in order if tr is not False]
            transposed = {}
            if need:
                joined = CtxtTensor(lib.batch_concat([x.ct for x in need]) if len(need) > 1 else need[0].ct, D, D, 2 * D)
                # schedule 2 transposes at the lowest level that leaves target + 3 for sigma / tau (transposeInplace's
                # own target_level argument, HEMMer.cpp:1166-1172); the other schedules transpose at the input level
                H.transpose_inplace(joined, t + 3 if getattr(H, "schedule", 0) == 2 else 0)
                pos = 0
                for tr in order:
                    if tr is False:
                        continue
                    cnt = len(cc[tr][0])
                    transposed[tr] = lib.batch_slice(joined.ct, pos, cnt) if len(need) > 1 else joined.ct
                    pos += cnt
            sas, tbs = [], []
            for tr in order:
                a = CtxtTensor(transposed[tr] if tr == "left" else cc[tr][1].ct, D, D, 2 * D)
                b = CtxtTensor(transposed[tr] if tr is True else cc[tr][2].ct, D, D, 2 * D)
                sa, tb = H.cc_matmul_prepare(a, b, t)
                sas.append(sa); tbs.append(tb)
            sa = lib.batch_concat(sas) if len(sas) > 1 else sas[0]
            tb = lib.batch_concat(tbs) if len(tbs) > 1 else tbs[0]
            out["ccmm"]["all"] = ([u for tr in order for u in cc[tr][0]], H.cc_matmul_core(sa, tb, D, D, D, 2 * D, t))
        return out

    def _reduce_partials(self, partial):
        """K-split exchange: every rank holds the partial products of its own K-groups; one all-reduce per sublayer
        (sum of residues, then reduction modulo each prime) gives every rank the complete output tiles -- the pattern of
        TransformerBlock::ncclAllReduceWrapper + modReduct (TransformerBlock.cpp:11142-11154, HEMMer.cpp:2625-2635)."""
        lib = self.lib
        for name, xname, weights, kt, nt in self.PCMM:
            keys = [(name, wname, j) for wname in weights for j in range(nt)]
            stacked = lib.ct_create(self.target + 1, 2, len(keys), 2)   # zero where this rank has no partial
            lib.ct_zero(stacked)
            for k, key in enumerate(keys):
                if key in partial:
                    lib.batch_set(stacked, k, partial[key].ct)
            lib.allreduce_sum(stacked, self.comm)
            for k, key in enumerate(keys):
                partial[key] = CtxtTensor(lib.batch_get(stacked, k), D, D, 2 * D)

    # ---- device -> host ----
    def _expected_ccmm(self, u):
        _, name, lhs, rhs, tr = u
        (a0, a1), (b0, b1) = self._pair(lhs), self._pair(rhs)
        if tr is True:
            b0, b1 = b0.T, b1.T
        elif tr == "left":
            a0, a1 = a0.T, a1.T
        return np.stack([a0 @ b0, a1 @ b1])

    def _decrypt_all(self, out, check=False):
        """Decrypt every result to host matrices (one batched call); returns the max-abs error when `check`."""
        err = 0.0
        per = 2 * self.lib.N * 8
        items, tags = [], []
        for k, ((name, wname, j), ct) in enumerate(out["pcmm"].items()):
            if k % self.world != self.rank:
                continue   # after the exchange every rank holds every output tile; each one is read back by one rank
            items.append((ct.ct, 0)); tags.append(("p", name, wname, j))
        for tr, (us, c) in out["ccmm"].items():
            for k, u in enumerate(us):
                items.append((c.ct, k)); tags.append(("c", u))
        if not items:
            return err
        zs = self.lib.decrypt_many(items)
        self.d2h_bytes += per * len(items)
        self.results = []
        for tag, z in zip(tags, zs):
            z = z[: D * 2 * D].reshape(D, 2 * D)
            if tag[0] == "p":
                got = 2 * (z[:, :D].real + z[:, D:].real)
                self.results.append(got)
                if check:
                    _, name, wname, j = tag
                    spec = [p for p in self.PCMM if p[0] == name][0]
                    x, w = self.data[spec[1]], self.data[wname]
                    err = max(err, float(np.abs(got - x[:, : spec[3] * D] @ w[: spec[3] * D, j * D:(j + 1) * D]).max()))
            else:
                self.results.append(z.real)
                if check:
                    exp = self._expected_ccmm(tag[1])
                    err = max(err, float(np.abs(z[:, :D].real - exp[0]).max()), float(np.abs(z[:, D:].real - exp[1]).max()))
        return err

    # ---- public steps ----
    def prepare(self):
        """Make every operand of this rank's units resident on the device."""
        self.resident = self._encrypt_all(10_000)

    def step_resident(self):
        return self._compute(self.resident)

    def step(self):
        return self._compute(self._encrypt_all(10_000))

    def step_e2e(self):
        """Host matrices in, decrypted host matrices out.  `phases_ms` accumulates the host-clock time of the three parts."""
        t0 = time.perf_counter()
        enc = self._encrypt_all(30_000)
        self.lib.sync()
        t1 = time.perf_counter()
        out = self._compute(enc)
        self.lib.sync()
        t2 = time.perf_counter()
        self._decrypt_all(out)
        t3 = time.perf_counter()
        for k, v in (("encode_encrypt", t1 - t0), ("compute", t2 - t1), ("decrypt_decode", t3 - t2)):
            self.phases_ms[k] = self.phases_ms.get(k, 0.0) + 1e3 * v
        return out

    def check(self):
        """Max-abs error of every result of this rank against the float64 products."""
        return self._decrypt_all(self._compute(self._encrypt_all(20_000)), check=True)
