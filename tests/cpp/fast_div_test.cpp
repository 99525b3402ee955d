// The multiply-and-shift division the general kernel flavour uses for its work-item arithmetic
// (tt-buda_b200/csrc/buda_common.cuh: fast_div_setup / fast_div) against the plain division, host side.
#include <cstdint>
#include <cstdio>
#include <random>

#include "buda_common.cuh"

int main()
{
    std::mt19937_64 rng(7);
    const uint32_t edge_n[] = {0u, 1u, 2u, 31u, 32u, 33u, 1023u, 4095u, 65535u, 65536u, 0x7ffffffeu, 0x7fffffffu};
    uint64_t checked = 0;
    for (int t = 0; t < 20000; t++) {
        uint32_t d = t < 4100 ? (uint32_t)t + 1u : (uint32_t)(rng() % 0x7fffffffu) + 1u;
        if (t % 7 == 0 && t > 4100) d = 1u << (rng() % 31);           // powers of two
        uint32_t magic;
        uint8_t shift;
        buda::fast_div_setup(d, magic, shift);
        for (uint32_t n : edge_n) {
            if (buda::fast_div(n, magic, shift) != n / d) { std::printf("FAILED n=%u d=%u\n", n, d); return 1; }
            checked++;
        }
        for (int k = 0; k < 64; k++) {
            uint32_t n = (uint32_t)(rng() & 0x7fffffffu);
            if (k < 8) n = (n / d) * d + (k < 4 ? 0u : d - 1u);         // multiples of d and the value just below the next one
            n &= 0x7fffffffu;
            if (buda::fast_div(n, magic, shift) != n / d) { std::printf("FAILED n=%u d=%u\n", n, d); return 1; }
            checked++;
        }
    }
    std::printf("ok %llu\n", (unsigned long long)checked);
    return 0;
}
