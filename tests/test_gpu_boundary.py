"""The drop-in boundary on the GPU: the HEMMer-level C entry points (encode / encrypt / decrypt of host matrices), the
file container, and the C++ class used from a separately compiled program."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT, MID, SMALL, rand_ct_residues

pytestmark = pytest.mark.gpu
PKG_DIR = os.path.join(ROOT, "encryption-friendly_llm_architecture_b200")


def _same(a, b, what=""):
    assert a.shape == b.shape and np.array_equal(a, b), what


def test_hemmer_entry_points_equal_the_layout_path(pkg, gpu_mid):
    """hb_hemmer_encode / encode2 / encodeDiagonalToRow4 / encrypt / encrypt2 / decrypt / decrypt2 (the C++ methods behind
    them) against the same layouts built in numpy and pushed through the primitive entry points."""
    from importlib import import_module
    hm = import_module("encryption-friendly_llm_architecture_b200.hemmer")
    g = gpu_mid
    H = pkg.open_hemmer(g)
    assert H._native("encode2") is not None, "the CUDA library's C++ layer must export the HEMMer-level entry points"
    d = 32
    rng = np.random.default_rng(8)
    A, B, W3, W4 = (rng.uniform(-1, 1, (d, d)) for _ in range(4))
    _same(g.pt_export(H.encode(A, 5).ct), g.pt_export(g.encode(hm.layout1(A, g.slots), 5)), "encode")
    _same(g.pt_export(H.encode2(A, B).ct), g.pt_export(g.encode(hm.layout2(A, B, g.slots), g.L)), "encode2 at the default level")
    _same(g.pt_export(H.encode_diagonal_to_row4(A, B, W3, W4, 4).ct), g.pt_export(g.encode(hm.layout_diag_to_row4(A, B, W3, W4, g.slots), 4)), "encodeDiagonalToRow4")
    c1, c2 = H.encrypt(A, nonce=11), H.encrypt2(A, B, nonce=12)
    _same(g.ct_export(c1.ct), g.ct_export(g.encrypt(g.encode(hm.layout1(A, g.slots), g.L), 11)), "encrypt")
    _same(g.ct_export(c2.ct), g.ct_export(g.encrypt(g.encode(hm.layout2(A, B, g.slots), g.L), 12)), "encrypt2")
    assert (c2.rows, c2.cols, c2.width) == (d, d, 2 * d)
    assert np.abs(H.decrypt(c1) - A).max() < 1e-6
    D = H.decrypt2(c2)
    assert D.shape == (2, d, d) and np.abs(D[0] - A).max() < 1e-6 and np.abs(D[1] - B).max() < 1e-6
    dll = H.dll
    assert dll.hb_hemmer_get_rank(H.h) == 0 and dll.hb_hemmer_get_max_rank(H.h) == 1
    assert dll.hb_hemmer_set_rank(H.h, C.c_int(3), C.c_int(8)) == 0 and dll.hb_hemmer_get_rank(H.h) == 3 and dll.hb_hemmer_get_max_rank(H.h) == 8
    assert dll.hb_hemmer_set_rank(H.h, C.c_int(8), C.c_int(8)) != 0


def test_files_round_trip(pkg, gpu_mid, tmp_path):
    """Ciphertext, plaintext and key files: what is loaded equals what was saved, in another context too; a file written
    under other parameters, a truncated one and one of the wrong kind are refused."""
    g = gpu_mid
    g.gen_rot_keys([1, 5])
    lvl = 6
    ct = g.ct_create(lvl, 2, 3)
    data = rand_ct_residues(g, lvl, 2, 3, seed=17)
    g.ct_import(ct, data)
    g.ct_save(ct, tmp_path / "a.bin")
    back = g.ct_load(tmp_path / "a.bin")
    assert g.ct_meta(back) == g.ct_meta(ct)
    _same(g.ct_export(back), data, "ciphertext file")
    z = np.random.default_rng(2).uniform(-1, 1, g.slots)
    for pt in (g.encode(z, 4), g.encode_ext(z, 3)):
        g.pt_save(pt, tmp_path / "p.bin")
        _same(g.pt_export(g.pt_load(tmp_path / "p.bin")), g.pt_export(pt), "plaintext file")
    keys = tmp_path / "keys"
    keys.mkdir()
    g.keys_save(keys)
    assert (keys / "SecretKey.bin").exists() and (keys / "MultKey.bin").exists() and (keys / f"GaloisKey_{g.galois(5)}.bin").exists()
    other = pkg.open_gpu(pkg.make_params(**MID))      # same parameters, no keys generated
    with pytest.raises(pkg.HBError):
        other.rotate(other.ct_load(tmp_path / "a.bin"), 5)
    other.keys_load(keys, [g.galois(1), g.galois(5), 2 * g.N - 1])
    theirs = other.ct_load(tmp_path / "a.bin")
    for op in (lambda L, x: L.rotate(x, 5), lambda L, x: L.conjugate(x), lambda L, x: L.relin(L.tensor(x, x))):
        _same(other.ct_export(op(other, theirs)), g.ct_export(op(g, ct)), "operation under reloaded keys")
    assert np.array_equal(other.decrypt(theirs, 1), g.decrypt(ct, 1))
    # refusals
    with pytest.raises(pkg.HBError):
        g.pt_load(tmp_path / "a.bin")                              # a ciphertext file is not a plaintext
    small = pkg.open_gpu(pkg.make_params(log_n=10, max_level=8, dnum=3, num_special=3, hamming_weight=32))
    with pytest.raises(pkg.HBError):
        small.ct_load(tmp_path / "a.bin")                          # other ring degree and primes
    raw = (tmp_path / "a.bin").read_bytes()
    (tmp_path / "cut.bin").write_bytes(raw[: len(raw) // 2])
    with pytest.raises(pkg.HBError):
        g.ct_load(tmp_path / "cut.bin")
    bad = bytearray(raw); bad[200] ^= 1
    (tmp_path / "flip.bin").write_bytes(bytes(bad))
    with pytest.raises(pkg.HBError):
        g.ct_load(tmp_path / "flip.bin")                           # checksum
    with pytest.raises(pkg.HBError):
        g.ct_load(tmp_path / "missing.bin")


def test_cpp_class_from_a_separately_compiled_program(pkg, tmp_path):
    """tests/integration/hemmer_snippet.cpp (the example of INTEGRATION.md) built with g++ against the two shared
    libraries, run, and compared with the same calls through ctypes: equal residues, correct products."""
    exe, out = tmp_path / "snippet", tmp_path / "snippet.bin"
    cmd = ["g++", "-O1", "-std=c++17", os.path.join(ROOT, "tests", "integration", "hemmer_snippet.cpp"), "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(PKG_DIR, "csrc", "hellm"), "-L", PKG_DIR, "-lhellm_b200", "-lhemmer_b200", f"-Wl,-rpath,{PKG_DIR}", "-o", str(exe)]
    subprocess.check_call(cmd)
    r = subprocess.run([str(exe), str(out)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    raw = out.read_bytes()
    level = int(np.frombuffer(raw[:4], dtype=np.int32)[0])
    d = 32
    mats = np.frombuffer(raw[4:4 + 8 * 6 * d * d], dtype=np.float64)
    x0, x1, w0, w1 = (mats[k * d * d:(k + 1) * d * d].reshape(d, d) for k in range(4))
    dec = mats[4 * d * d:].reshape(2, d, d)
    residues = np.frombuffer(raw[4 + 8 * 6 * d * d:], dtype=np.uint64).reshape(1, 2, level + 1, 4096)
    assert level == 3
    assert np.abs(dec[0] - x0 @ w0).max() < 2.0 ** -14 and np.abs(dec[1] - x1 @ w1).max() < 2.0 ** -14
    g = pkg.open_gpu(pkg.make_params(**MID))
    g.keygen()
    H = pkg.open_hemmer(g)
    c = H.single_cc_matmul(H.encrypt2(x0, x1, nonce=1), H.encrypt2(w0, w1, nonce=2), 3)
    _same(g.ct_export(c.ct), residues, "C++ program and ctypes path")


def test_bounded_wait_gives_up_and_reports_timeout(pkg):
    """A device-side wait that nothing completes runs out of polls, raises the context's flag and returns: the next
    sync reports HB_E_TIMEOUT (-8) once, and the context computes correctly afterwards."""
    g = pkg.open_gpu(pkg.make_params(**SMALL))
    g.keygen()
    assert g.dll.hb_selftest_bounded_wait(g.ctx) == 0
    assert g.dll.hb_sync(g.ctx) == -8
    assert b"bounded wait" in g.dll.hb_last_error(g.ctx)
    assert g.dll.hb_sync(g.ctx) == 0
    z = np.random.default_rng(3).uniform(-1, 1, g.slots)
    ct = g.encrypt(g.encode(z, g.L), 7)
    assert np.abs(g.decrypt(ct).real - z).max() < 2.0 ** -14


def test_release_cached_returns_idle_buffers(pkg):
    g = pkg.open_gpu(pkg.make_params(**SMALL))
    g.keygen()
    z = np.random.default_rng(4).uniform(-1, 1, g.slots)
    ct = g.encrypt(g.encode(z, g.L), 9)
    tmp = g.rescale(g.mul_pt_norescale(ct, g.encode(z, g.L)))
    del tmp
    pool, used = C.c_uint64(), C.c_uint64()
    g.dll.hb_mem_info(g.ctx, C.byref(pool), C.byref(used))
    before = pool.value
    assert g.dll.hb_release_cached(g.ctx) == 0
    g.dll.hb_mem_info(g.ctx, C.byref(pool), C.byref(used))
    assert pool.value < before and pool.value >= used.value
    assert np.abs(g.decrypt(ct).real - z).max() < 2.0 ** -14
