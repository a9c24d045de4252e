"""Pins for the CPU oracle: identities that hold independently of the oracle's own code."""
import ctypes as C

import numpy as np
import pytest

from conftest import open_oracle

TOL = 2.0 ** -14  # the reference's comparison tolerance (ciphertext/test/HELLMTestBase.hpp:34)


def test_chacha20_block_rfc8439(pkg, oracle_so):
    """RFC 8439 section 2.3.2 block-function test vector."""
    dll = C.CDLL(oracle_so)
    key = (C.c_uint32 * 8)(*[int.from_bytes(bytes(range(4 * i, 4 * i + 4)), "little") for i in range(8)])
    nonce = (C.c_uint32 * 3)(0x09000000, 0x4A000000, 0x00000000)
    out = (C.c_uint32 * 16)()
    dll.orc_chacha_block(key, C.c_uint32(1), nonce, out)
    expect = [0xE4E7F110, 0x15593BD1, 0x1FDD0F50, 0xC47120A3, 0xC7F4D1C7, 0x0368C033, 0x9AAA2204, 0x4E6CD4C3,
              0x466482D2, 0x09AA9F07, 0x05D7C214, 0xA2028BD9, 0xD19C12B5, 0xB94E16DE, 0xE883D0CB, 0x4E3C50A2]
    assert list(out) == expect


@pytest.fixture(scope="module")
def tiny(pkg, oracle_so):
    o = open_oracle(pkg, oracle_so, log_n=4, max_level=3, dnum=3, num_special=2, hamming_weight=4)
    o.keygen()
    return o


def test_prime_chain(tiny, orc_small):
    for o in (tiny, orc_small):
        for q in o.primes:
            q = int(q)
            assert q % (2 * o.N) == 1
            assert all(q % p for p in (3, 5, 7, 11, 13)) and pow(2, q - 1, q) == 1
        assert len(set(int(q) for q in o.primes)) == len(o.primes)
        # scale ladder: Delta_{l-1} = Delta_l^2 / q_l
        for l in range(o.L, 0, -1):
            assert o.scales[l - 1] == o.scales[l] * o.scales[l] / float(o.primes[l])


def _ntt(o, a, prime_index, inverse=False):
    buf = np.ascontiguousarray(a, dtype=np.uint64).copy()
    o.dll.orc_ntt_limb(o.ctx, buf.ctypes.data_as(C.POINTER(C.c_uint64)), C.c_int(prime_index), C.c_int(1 if inverse else 0))
    return buf


def _bitrev(x, bits):
    return int(format(x, f"0{bits}b")[::-1], 2)


def test_ntt_is_evaluation_at_odd_powers(tiny):
    """a_hat[i] = a(psi^(2*bitrev(i)+1)), checked with Python integers."""
    o = tiny
    o.dll.orc_psi.restype = C.c_uint64
    rng = np.random.default_rng(1)
    for pi in range(len(o.primes)):
        q = int(o.primes[pi])
        psi = int(o.dll.orc_psi(o.ctx, C.c_int(pi)))
        assert pow(psi, o.N, q) == q - 1
        a = [int(x) for x in rng.integers(0, q, o.N, dtype=np.uint64)]
        got = _ntt(o, np.array(a, dtype=np.uint64), pi)
        for i in range(o.N):
            x = pow(psi, 2 * _bitrev(i, 4) + 1, q)
            assert int(got[i]) == sum(c * pow(x, k, q) for k, c in enumerate(a)) % q
        back = _ntt(o, got, pi, inverse=True)
        assert [int(v) for v in back] == a


def test_ntt_product_is_negacyclic_schoolbook(orc_small):
    o = orc_small
    rng = np.random.default_rng(2)
    q = int(o.primes[1])
    n = o.N
    a = [int(x) for x in rng.integers(0, q, n, dtype=np.uint64)]
    b = [int(x) for x in rng.integers(0, q, n, dtype=np.uint64)]
    # sparse b keeps the schoolbook product cheap
    for k in range(n):
        if k % 37:
            b[k] = 0
    ref = [0] * n
    for j, bj in enumerate(b):
        if not bj:
            continue
        for i, ai in enumerate(a):
            k = i + j
            if k < n:
                ref[k] = (ref[k] + ai * bj) % q
            else:
                ref[k - n] = (ref[k - n] - ai * bj) % q
    fa = _ntt(o, np.array(a, dtype=np.uint64), 1)
    fb = _ntt(o, np.array(b, dtype=np.uint64), 1)
    prod = np.array([int(x) * int(y) % q for x, y in zip(fa, fb)], dtype=np.uint64)
    assert [int(v) for v in _ntt(o, prod, 1, inverse=True)] == ref


def test_encode_is_canonical_embedding(tiny):
    """Decoding evaluates the plaintext polynomial at zeta^(5^j), zeta = exp(i pi / N)."""
    o = tiny
    rng = np.random.default_rng(3)
    z = rng.uniform(-1, 1, o.slots) + 1j * rng.uniform(-1, 1, o.slots)
    pt = o.encode(z, o.L)
    res = o.pt_export(pt)
    coeff = _ntt(o, res[0], 0, inverse=True).astype(object)
    q0 = int(o.primes[0])
    coeff = [int(c) - q0 if int(c) > q0 // 2 else int(c) for c in coeff]
    zeta = np.exp(1j * np.pi / o.N)
    for j in range(o.slots):
        x = zeta ** pow(5, j, 2 * o.N)
        val = sum(c * x ** k for k, c in enumerate(coeff)) / o.scales[o.L]
        assert abs(val - z[j]) < 1e-9
    assert np.abs(o.decode(pt) - z).max() < 1e-9


def test_automorphism_permutation_matches_rotation(orc_small):
    o = orc_small
    g = o.galois(3)
    perm = np.zeros(o.N, dtype=np.uint32)
    o.dll.orc_ntt_perm(o.ctx, C.c_uint64(g), perm.ctypes.data_as(C.POINTER(C.c_uint32)))
    assert sorted(perm.tolist()) == list(range(o.N))
    rng = np.random.default_rng(4)
    z = rng.uniform(-1, 1, o.slots)
    pt = o.encode(z, 2)
    res = o.pt_export(pt)
    # a permuted plaintext decodes to the rotated message
    ct = o.ct_create(2, 1, 1)
    o.ct_import(ct, res[:, perm].reshape(1, 1, 3, o.N))
    zero = o.ct_create(2, 2, 1)
    buf = np.zeros((1, 2, 3, o.N), dtype=np.uint64)
    buf[0, 0] = res[:, perm]
    o.ct_import(zero, buf)
    assert np.abs(o.decrypt(zero).real - np.roll(z, -3)).max() < 1e-8


def test_primitives_semantics(orc_small):
    o = orc_small
    o.gen_rot_keys([1, 5, -7])
    rng = np.random.default_rng(5)
    z = rng.uniform(-1, 1, o.slots) + 1j * rng.uniform(-1, 1, o.slots)
    w = rng.uniform(-1, 1, o.slots)
    cz = o.encrypt(o.encode(z, o.L), 11)
    cw = o.encrypt(o.encode(w, o.L), 12)
    tol = 1e-6
    assert np.abs(o.decrypt(cz) - z).max() < tol
    assert np.abs(o.decrypt(o.add(cz, cw)) - (z + w)).max() < tol
    assert np.abs(o.decrypt(o.sub(cz, cw)) - (z - w)).max() < tol
    assert np.abs(o.decrypt(o.negate(cz)) + z).max() < tol
    assert np.abs(o.decrypt(o.mult_imag(cz)) - 1j * z).max() < tol
    assert np.abs(o.decrypt(o.mult_int(cz, -3)) + 3 * z).max() < tol
    assert np.abs(o.decrypt(o.mul(cz, cw)) - z * w).max() < tol
    assert np.abs(o.decrypt(o.mul_pt(cz, o.encode(w, o.L))) - z * w).max() < tol
    for s in (1, 5, -7):
        assert np.abs(o.decrypt(o.rotate(cz, s)) - np.roll(z, -s)).max() < tol
    assert np.abs(o.decrypt(o.conjugate(cz)) - np.conj(z)).max() < tol
    low = o.level_down(cz, 2)
    assert o.ct_meta(low)[0] == 2 and np.abs(o.decrypt(low) - z).max() < tol
    # level-adjusting add
    mixed = o.add(o.mul(cz, cw), cz)
    assert o.ct_meta(mixed)[0] == o.L - 1 and np.abs(o.decrypt(mixed) - (z * w + z)).max() < tol
    # tensor without relinearisation still decrypts (three-poly ciphertext, scale Delta^2)
    t = o.tensor(cz, cw)
    assert o.ct_meta(t) == (o.L, 3, 1, 2) and np.abs(o.decrypt(t) - z * w).max() < tol
    assert np.abs(o.decrypt(o.rescale(o.relin(t))) - z * w).max() < tol


def test_rescale_is_exact_rounded_division(orc_small):
    """rescale divides the underlying integer polynomial by q_l with rounding: check through decryption of a plaintext-like ciphertext (a = 0)."""
    o = orc_small
    lvl = 3
    rng = np.random.default_rng(6)
    ql = int(o.primes[lvl])
    coeffs = [int(x) for x in rng.integers(-2 ** 50, 2 ** 50, o.N)]
    buf = np.zeros((1, 2, lvl + 1, o.N), dtype=np.uint64)
    for l in range(lvl + 1):
        q = int(o.primes[l])
        buf[0, 0, l] = _ntt(o, np.array([c % q for c in coeffs], dtype=np.uint64), l)
    ct = o.ct_create(lvl, 2, 1, 2)
    o.ct_import(ct, buf)
    out = o.ct_export(o.rescale(ct))
    for l in range(lvl):
        q = int(o.primes[l])
        got = [int(v) for v in _ntt(o, out[0, 0, l], l, inverse=True)]
        for c, g in zip(coeffs[:64], got[:64]):
            r = c % ql
            if r > ql // 2:
                r -= ql
            assert g == ((c - r) // ql) % q


def test_keyswitch_base_conversion_against_bigint(pkg, oracle_so):
    """Rotation key switching at tiny N: the result decrypts to the rotated message with noise far below the tolerance,
    at every level (which exercises partial last digits)."""
    o = open_oracle(pkg, oracle_so, log_n=6, max_level=7, dnum=3, num_special=3, hamming_weight=8)
    o.keygen()
    o.gen_rot_keys([1])
    z = np.random.default_rng(7).uniform(-1, 1, o.slots)
    ct = o.encrypt(o.encode(z, o.L), 3)
    for lvl in range(o.L, -1, -1):
        c = o.level_down(ct, lvl)
        assert np.abs(o.decrypt(o.rotate(c, 1)).real - np.roll(z, -1)).max() < 1e-6, lvl
