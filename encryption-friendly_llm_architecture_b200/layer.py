"""BERT-base encoder-layer matmul workload over HEMMer (forward + LoRA backward), tile-sharded.

Shapes follow the reference's micro-benchmarks (ciphertext/examples/bert-matmul.cpp,
bert-matmul-backward.cpp): 128 tokens, hidden 768 = 6 tiles of 128, FFN 3072 = 24 tiles, two tiles per
ciphertext ([A | B], HEMMer::encrypt2), plaintext weights packed four tiles per plaintext
(HEMMer::encodeDiagonalToRow4).  As in those programs every matmul starts from freshly encrypted
top-level operands; the non-linear steps between them (softmax, layer norm, bootstrapping) are not
part of the workload.

Work items are independent "units" (one matMulPre group with its matMulReUse products, or one
two-tile ct x ct product).  Units are dealt to the ranks by estimated cost (longest first, to the least
loaded rank), so the same code runs on 1..8 GPUs.  The K-groups of one ct x pt sublayer may sit on
different ranks: every output tile then has one owner among those ranks, the others send it their
partial products, and the owner adds them up modulo each prime (the role of
TransformerBlock::ncclReduceWrapper + modReduct, TransformerBlock.cpp:11100-11140).

The encryption randomness of a unit depends on the unit's position in the layer only, never on the rank
count, and all sums are exact modular sums: every rank count produces the same ciphertext bits.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import time

import numpy as np

from .hemmer import CtxtTensor, Hemmer

D = 128          # tile side
HIDDEN = 6       # 768 / 128
FFN = 24         # 3072 / 128
HEADS = 12
LORA_RANK = 8

# Device time of one unit of each cost class in milliseconds, fitted to the per-rank times of an 8-GPU pass on B200s
# (ranks with different mixes of units; batching makes the figures marginal costs, and only their ratios matter).
UNIT_COST_MS = {"qkv": 18.5, "wo": 11.8, "w1": 20.2, "w2": 12.6, "ccmm": 16.3, "ccmm_t": 19.0}


def synthetic(seed: int):
    """Seeded inputs with the distributions of the workload definition: activations U[-1,1], weights N(0, 0.02^2),
    attention scores U[0, 1/128]."""
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


def unit_kind(u):
    """Cost class of a unit: the ct x pt sublayer, or ct x ct with / without a transpose."""
    return u[1] if u[0] == "pcmm" else ("ccmm_t" if u[4] else "ccmm")


def unit_cost(u):
    return UNIT_COST_MS[unit_kind(u)]


def deal_units(units, world):
    """Owner rank of every unit: longest estimated time first, each to the rank with the least work so far."""
    load = [0.0] * world
    owner = [0] * len(units)
    for i in sorted(range(len(units)), key=lambda i: (-unit_cost(units[i]), i)):
        r = min(range(world), key=lambda r: (load[r], r))
        owner[i] = r
        load[r] += unit_cost(units[i])
    return owner


def sha(arr):
    return hashlib.sha256(np.ascontiguousarray(arr, dtype=np.uint64).tobytes()).hexdigest()


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
        self.owner = deal_units(self.units, world)
        self.mine = [i for i in range(len(self.units)) if self.owner[i] == rank]
        # canonical list of ct x pt output tiles and, per sublayer, the ranks that hold partial products of them
        self.tile_keys = [(name, wname, j) for name, _, weights, _, nt in self.PCMM for wname in weights for j in range(nt)]
        self.members = {name: sorted({self.owner[i] for i, u in enumerate(self.units) if u[0] == "pcmm" and u[1] == name}) for name, *_ in self.PCMM}
        self.tile_owner = {}
        for name, _, weights, _, nt in self.PCMM:
            keys = [(name, wname, j) for wname in weights for j in range(nt)]
            for k, key in enumerate(keys):
                self.tile_owner[key] = self.members[name][k % len(self.members[name])]
        self.h2d_bytes = 0
        self.phases_ms = {}
        self.d2h_bytes = 0
        self.comm_events = []   # (start, end) CUDA event pairs around the exchange, filled by bench.py's hooks
        self.on_comm = None     # optional callable(phase) -> None, phase in {"start", "end"}
        self._weights = {}
        self.resident = None
        self.comm = None        # NCCL communicator (void*) when several ranks split the K-groups of a sublayer

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

    def unit_index(self, name, g=None):
        for i, u in enumerate(self.units):
            if u[1] == name and (u[0] == "ccmm" or u[4] == g):
                return i
        raise KeyError((name, g))

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

    def _x_pairs(self, u):
        """The one or two [A | B] operand pairs of a ct x pt unit."""
        _, name, xname, weights, g, kt, nt = u
        x = self.data[xname]
        pair = lambda p: (tiles(x, 0, 2 * p), tiles(x, 0, 2 * p + 1))
        ops = [pair(2 * g)]
        if 4 * g + 2 < kt:
            ops.append(pair(2 * g + 1))
        return ops

    def _weight_pts(self, wname, g, kt, nt, only=None):
        key = (wname, g)
        if only is not None:   # one plaintext, not cached (the single-unit path)
            w = self.data[wname]
            z = np.zeros((D, D))
            t = [tiles(w, 4 * g + i, only) if 4 * g + i < kt else z for i in range(4)]
            return self.H.encode_diagonal_to_row4(*t, level=self.target + 1)
        if key not in self._weights:
            w = self.data[wname]
            z = np.zeros((D, D))
            pts = []
            for j in range(nt):
                t = [tiles(w, 4 * g + i, j) if 4 * g + i < kt else z for i in range(4)]
                pts.append(self.H.encode_diagonal_to_row4(*t, level=self.target + 1))
            self._weights[key] = pts
        return self._weights[key]

    def _transpose_target(self):
        # schedule 2 transposes at the lowest level that leaves target + 3 for sigma / tau (transposeInplace's own
        # target_level argument, HEMMer.cpp:1166-1172); the other schedules transpose at the input level
        return self.target + 3 if getattr(self.H, "schedule", 0) == 2 else 0

    # ---- one unit on its own, through the plain (unbatched) calls: what every batch member must equal ----
    def ccmm_alone(self, i, nonce0):
        """Result handle of ct x ct unit i computed by itself (HEMMer::encrypt2, transposeInplace, singleCCMatMul)."""
        H, t = self.H, self.target
        _, name, lhs, rhs, tr = self.units[i]
        a = H.encrypt2(*self._pair(lhs), nonce=nonce0 + 2 * i)
        b = H.encrypt2(*self._pair(rhs), nonce=nonce0 + 2 * i + 1)
        if tr is True:
            H.transpose_inplace(b, self._transpose_target())
        elif tr == "left":
            H.transpose_inplace(a, self._transpose_target())
        return H.single_cc_matmul(a, b, t)

    def pcmm_tile_alone(self, key, nonce0):
        """Output tile (sublayer, weight, j) computed by itself: complexPacking + matMulPre + matMulReUse per K-group,
        partial products added (bert-matmul.cpp:251-293 without the repack)."""
        H, t = self.H, self.target
        name, wname, j = key
        acc = None
        for i, u in enumerate(self.units):
            if u[0] != "pcmm" or u[1] != name:
                continue
            ops = self._x_pairs(u)
            cts = [H.encrypt2(*p, nonce=nonce0 + 2 * i + k) for k, p in enumerate(ops)]
            packed = H.complex_packing(cts[0], cts[1]) if len(cts) == 2 else cts[0]
            part = H.matmul_reuse(H.matmul_pre(packed, t), self._weight_pts(wname, u[4], u[5], u[6], only=j))
            acc = part if acc is None else CtxtTensor(self.lib.add(acc.ct, part.ct), *part.shape)
        return acc

    # ---- host -> device ----
    def _encrypt_all(self, nonce0):
        """Encode + encrypt every operand of this rank's units, one batched call per group of operands."""
        H, lib = self.H, self.lib
        per_ct = 2 * lib.N * 8  # rounded message coefficients + error polynomial uploaded per encryption
        groups = {"full": [], "half": []}      # pcmm: (unit index, [(pair, nonce)])
        ccmm = {False: [], True: [], "left": []}
        for i in self.mine:
            u = self.units[i]
            n = nonce0 + 2 * i                 # the randomness of a unit does not depend on the rank count
            if u[0] == "pcmm":
                _, name, xname, weights, g, kt, nt = u
                ops = [(p, n + k) for k, p in enumerate(self._x_pairs(u))]
                self.h2d_bytes += per_ct * len(ops)
                for wname in weights:
                    self._weight_pts(wname, g, kt, nt)
                groups["full" if len(ops) == 2 else "half"].append((i, ops))
            else:
                _, name, lhs, rhs, tr = u
                self.h2d_bytes += 2 * per_ct
                ccmm[tr].append((i, (self._pair(lhs), n), (self._pair(rhs), n + 1)))
        many = lambda ops: H.encrypt2_many([p for p, _ in ops], [k for _, k in ops])
        res = {"pcmm": {}, "ccmm": {}}
        for kind, lst in groups.items():
            if lst:
                res["pcmm"][kind] = ([i for i, _ in lst], many([o[0] for _, o in lst]),
                                     many([o[1] for _, o in lst]) if kind == "full" else None)
        for tr, lst in ccmm.items():
            if lst:
                res["ccmm"][tr] = ([i for i, _, _ in lst], many([a for _, a, _ in lst]), many([b for _, _, b in lst]))
        return res

    # ---- device work ----
    def _compute(self, res):
        H, t = self.H, self.target
        out = {"pcmm": {}, "ccmm": {}}
        pres = {}
        for kind, (idx, c01, c23) in res["pcmm"].items():
            packed = H.complex_packing(c01, c23) if c23 is not None else c01
            pres[kind] = (idx, H.matmul_pre(packed, t))
        # every (sublayer, weight, output tile): one fused pass per batch of K-groups, partial sums added
        # (all output tiles of a sublayer meet the same shifted copies: one call per sublayer and kind of copies)
        for name, xname, weights, kt, nt in self.PCMM:
            tags = [(wname, j) for wname in weights for j in range(nt)]
            accs = [None] * len(tags)
            for kind, (idx, pre) in pres.items():
                sel = [(b, self.units[i]) for b, i in enumerate(idx) if self.units[i][1] == name]
                if not sel:
                    continue
                b0 = sel[0][0]
                by_tile = [[self._weight_pts(wname, u[4], kt, nt)[j] for _, u in sel] for wname, j in tags]
                parts = H.matmul_reuse_groups_tiles(pre, len(idx), b0, by_tile)
                for k, part in enumerate(parts):
                    accs[k] = part if accs[k] is None else CtxtTensor(self.lib.add(accs[k].ct, part.ct), *part.shape)
            for (wname, j), acc in zip(tags, accs):
                if acc is not None:
                    out["pcmm"][(name, wname, j)] = acc
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
                H.transpose_inplace(joined, self._transpose_target())
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
            out["ccmm"]["all"] = ([i for tr in order for i in cc[tr][0]], H.cc_matmul_core(sa, tb, D, D, D, 2 * D, t))
        # the K-split exchange comes last: a rank that finishes its own units early waits for its peers once, at the
        # end of the pass, instead of in the middle of it
        if self.world > 1:
            self._exchange_partials(out["pcmm"])
        return out

    def exchange_plan(self):
        """Transfers of the K-split exchange in the order every rank issues them: (tile key, source rank, owner rank)."""
        plan = []
        for key in self.tile_keys:
            mem, own = self.members[key[0]], self.tile_owner[key]
            plan += [(key, m, own) for m in mem if m != own]
        return plan

    def _exchange_partials(self, partial):
        """K-split exchange.  A sublayer's K-groups sit on the ranks `members[sublayer]`; each of its output tiles has one
        owner among them.  Inside one NCCL group every other member sends the owner its partial product; the owner then
        adds its own and the received ones and reduces modulo each prime in one pass.  Afterwards `partial` holds, on
        every rank, exactly the tiles this rank owns."""
        lib, rank = self.lib, self.rank
        if self.on_comm:
            self.on_comm("start")
        recv = {}
        lib.nccl_group_start()
        for key, src, own in self.exchange_plan():
            if rank == src:
                lib.send(partial[key].ct, own, self.comm)
            elif rank == own:
                buf = lib.ct_create(self.target + 1, 2, 1, 2)
                lib.recv(buf, src, self.comm)
                recv.setdefault(key, []).append(buf)
        lib.nccl_group_end()
        for key in list(partial):
            if self.tile_owner[key] != rank:
                del partial[key]
            elif key in recv:
                partial[key] = CtxtTensor(lib.sum_mod_reduce([partial[key].ct] + recv[key]), D, D, 2 * D)
        if self.on_comm:
            self.on_comm("end")

    # ---- device -> host ----
    def _expected_ccmm(self, u):
        _, name, lhs, rhs, tr = u
        (a0, a1), (b0, b1) = self._pair(lhs), self._pair(rhs)
        if tr is True:
            b0, b1 = b0.T, b1.T
        elif tr == "left":
            a0, a1 = a0.T, a1.T
        return np.stack([a0 @ b0, a1 @ b1])

    def held_outputs(self, out):
        """(tag, handle, batch index) of every result this rank holds after the exchange, in canonical order.  Tags:
        ("p", sublayer, weight, j) for ct x pt output tiles, ("c", unit index) for ct x ct products."""
        items = []
        for key in self.tile_keys:
            if key in out["pcmm"] and self.tile_owner[key] == self.rank:
                items.append((("p",) + key, out["pcmm"][key].ct, 0))
        for _, (idx, c) in out["ccmm"].items():
            for k, i in enumerate(idx):
                items.append((("c", i), c.ct, k))
        return items

    def output_digests(self, out):
        """SHA-256 of the residues of every result this rank holds: {tag: hex digest}."""
        lib = self.lib
        dig = {}
        cache = {}
        for tag, ct, k in self.held_outputs(out):
            if id(ct) not in cache:
                cache[id(ct)] = lib.ct_export(ct)
            dig[tag] = sha(cache[id(ct)][k])
        return dig

    def _decrypt_all(self, out, check=False):
        """Decrypt every result this rank holds to host matrices (one batched call); returns the max-abs error when `check`."""
        err = 0.0
        per = 2 * self.lib.N * 8
        held = self.held_outputs(out)
        if not held:
            return err
        zs = self.lib.decrypt_many([(ct, k) for _, ct, k in held])
        self.d2h_bytes += per * len(held)
        self.results = []
        for (tag, _, _), z in zip(held, zs):
            z = z[: D * 2 * D].reshape(D, 2 * D)
            if tag[0] == "p":
                got = 2 * (z[:, :D].real + z[:, D:].real)
                self.results.append((tag, got))
                if check:
                    _, name, wname, j = tag
                    spec = [p for p in self.PCMM if p[0] == name][0]
                    x, w = self.data[spec[1]], self.data[wname]
                    err = max(err, float(np.abs(got - x[:, : spec[3] * D] @ w[: spec[3] * D, j * D:(j + 1) * D]).max()))
            else:
                self.results.append((tag, z.real))
                if check:
                    exp = self._expected_ccmm(self.units[tag[1]])
                    err = max(err, float(np.abs(z[:, :D].real - exp[0]).max()), float(np.abs(z[:, D:].real - exp[1]).max()))
        return err

    # ---- public steps ----
    def prepare(self):
        """Make every operand of this rank's units resident on the device."""
        self.resident = self._encrypt_all(10_000)

    def step_resident(self):
        return self._compute(self.resident)

    def record_graph(self):
        """Record one resident pass as a CUDA graph (after at least one ordinary pass).  Returns (graph handle, results of
        the recorded pass); each replay recomputes those results in place from the resident operands."""
        lib = self.lib
        lib.graph_begin()
        try:
            out = self._compute(self.resident)
        finally:
            g = lib.graph_end()
        return g, out

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

    def check(self, with_digests=False):
        """Max-abs error of every result of this rank against the float64 products (and, on request, the digests of the
        same results: {tag: sha256})."""
        out = self._compute(self._encrypt_all(20_000))
        err = self._decrypt_all(out, check=True)
        return (err, self.output_digests(out)) if with_digests else err
