// Fuzz driver for the packet path of the C ABI (csrc/core/c_api.cpp), meant to be built with
// -fsanitize=address,undefined: a sender and a receiver hook exchange packets of random gradients (with the
// odd inf / NaN), and the receiver is handed intact, bit-flipped, truncated, over-long and random packets and
// wrong element counts. The library must answer every one of them with a return code; the sanitizers watch the
// memory. Prints "accepted A rejected R" at the end.
//
//   ffi_fuzz [trials per mode]
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include "nangila_ffi.h"

int main(int argc, char** argv) {
    const int trials = argc > 1 ? std::atoi(argv[1]) : 1000;
    std::mt19937_64 rng(12345);
    const size_t n = 1000;
    std::vector<float> g(n), out(n);
    int rejected = 0, accepted = 0;
    for (int mode = 0; mode < 2; ++mode) {  // with and without warm-up steps
        NangilaHandle tx = nangila_init_all_drivers_ex(2, mode ? 0 : 3, 0), rx = nangila_init_all_drivers_ex(2, mode ? 0 : 3, 0);
        std::vector<uint8_t> pkt(nangila_max_compressed_size(n));
        for (int t = 0; t < trials; ++t) {
            for (auto& v : g) v = float(int(rng() % 2001) - 1000) * 1e-4f;
            if (t % 50 == 7) g[rng() % n] = 1e38f * 100.0f;
            if (t % 50 == 9) g[rng() % n] = 0.0f / 0.0f;
            size_t sz = pkt.size();
            if (nangila_compress(tx, g.data(), n, uint32_t(t % 2), pkt.data(), &sz) != 0 || sz > pkt.size()) { std::printf("compress failed\n"); return 1; }
            std::vector<uint8_t> bad(pkt.begin(), pkt.begin() + long(sz));
            switch (rng() % 6) {
                case 0: break;
                case 1: bad[rng() % bad.size()] ^= uint8_t(1 + rng() % 255); break;
                case 2: bad.resize(rng() % bad.size()); break;
                case 3: for (int k = 0; k < 8 && !bad.empty(); ++k) bad[rng() % bad.size()] = 0xFF; break;
                case 4: bad.insert(bad.end(), 64, 0xAB); break;
                default: for (auto& b : bad) b = uint8_t(rng()); break;
            }
            const size_t count = (rng() % 8 == 0) ? size_t(rng() % (2 * n)) : n;
            std::vector<float> recv(count ? count : 1);
            if (nangila_decompress(rx, bad.data(), bad.size(), uint32_t(t % 2), recv.data(), count) == 0) {
                ++accepted;
                nangila_on_complete(rx, recv.data(), count, uint32_t(t % 2));
            } else {
                ++rejected;
            }
            if (nangila_decompress(tx, pkt.data(), sz, uint32_t(t % 2), out.data(), n) == 0) nangila_on_complete(tx, out.data(), n, uint32_t(t % 2));
            nangila_step(tx);
            nangila_step(rx);
        }
        nangila_free(tx);
        nangila_free(rx);
    }
    NangilaHandle h = nangila_init_all_drivers(1);
    size_t sz = 0;
    uint8_t small[4] = {0, 0, 0, 0};
    if (nangila_compress(nullptr, g.data(), n, 0, small, &sz) == 0 || nangila_compress(h, nullptr, n, 0, small, &sz) == 0 ||
        nangila_decompress(h, small, 4, 99, out.data(), n) == 0) { std::printf("a bad call was accepted\n"); return 1; }
    nangila_free(h);
    nangila_free(nullptr);
    std::printf("accepted %d rejected %d\n", accepted, rejected);
    return 0;
}
