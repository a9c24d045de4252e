// The C++ usage example of INTEGRATION.md, section 1, as a program: HELLM::HEMMer of this repository used the way the
// reference's examples use theirs (ciphertext/examples/bert-matmul.cpp:142-160, 452-470).  It writes the residues of
// the product and the decrypted matrices to the file named on the command line, so that a test can compare them with
// the same calls made through the C ABI from another language.
#include "HEMMer.hpp"

#include <cstdio>
#include <random>
#include <vector>

int main(int argc, char **argv) {
    if (argc < 2) return 2;
    const int d = 32;                                       // tile side for N = 2^12 (two tiles fill the 2048 slots)
    hb_params prm = {12, 8, 3, 3, 60, 42, 60, 64, 3.2, {0x243F6A8885A308D3ull, 0x13198A2E03707344ull, 0xA4093822299F31D0ull, 0x082EFA98EC4E6C89ull}};
    HELLM::HEMMer *hemmer = HELLM::HEMMer::genHEMMer(/*device*/ 0, prm);
    std::mt19937_64 rng(5);
    std::uniform_real_distribution<double> u(-1.0, 1.0);
    std::vector<double> x0(d * d), x1(d * d), w0(d * d), w1(d * d), out(2 * d * d);
    for (auto *v : {&x0, &x1, &w0, &w1})
        for (double &e : *v) e = u(rng);
    auto a = hemmer->encrypt2(x0.data(), x1.data(), d, d, /*nonce*/ 1);
    auto b = hemmer->encrypt2(w0.data(), w1.data(), d, d, 2);
    auto c = hemmer->singleCCMatMul(a, b, /*target_level*/ 3);
    hemmer->decrypt2(c, out.data());                       // [2][d][d] doubles
    std::vector<uint64_t> residues((size_t)2 * (c.getLevel() + 1) * 4096);
    HELLM::check(hemmer->context(), hb_ct_export(hemmer->context(), c.get().raw(), residues.data()));
    FILE *f = std::fopen(argv[1], "wb");
    if (!f) return 3;
    const int level = c.getLevel();
    std::fwrite(&level, sizeof(level), 1, f);
    for (auto *v : {&x0, &x1, &w0, &w1, &out}) std::fwrite(v->data(), sizeof(double), v->size(), f);
    std::fwrite(residues.data(), 8, residues.size(), f);
    std::fclose(f);
    delete hemmer;
    std::printf("ok level %d\n", level);
    return 0;
}
