// Host-side check of the EXL3 window extraction used by the CUDA kernels (exl3_decode.cuh, lane_states<K>) against
// the plain definition of the format: state t = ring bits [t*K+K-16, t*K+K) of the tile read MSB-first.
// Built with nvcc and run on the CPU by tests/test_host_logic.py; no GPU is involved.
#include <cstdio>
#include <cstdint>
#include <cstdlib>
#include "../exllamav3-rs_b200/csrc/exl3_decode.cuh"

static uint32_t ring_state(const uint32_t* w, int K, int t)
{
    const int L = 256 * K;
    uint32_t s = 0;
    for (int i = 0; i < 16; ++i) {
        int bit = ((t * K + K - 16 + i) % L + L) % L;       // bit index from the MSB of word 0
        s = (s << 1) | ((w[bit >> 5] >> (31 - (bit & 31))) & 1u);
    }
    return s;
}

template <int K> int check()
{
    int bad = 0;
    uint32_t w[64];
    for (int rep = 0; rep < 50; ++rep) {
        for (int i = 0; i < 8 * K; ++i) w[i] = ((uint32_t)rand() << 17) ^ ((uint32_t)rand() << 3) ^ (uint32_t)rand();
        for (int lane = 0; lane < 32; ++lane) {
            uint32_t st[8];
            exl3::lane_states<K>(w, lane, st);
            for (int j = 0; j < 8; ++j)
                if (st[j] != ring_state(w, K, 8 * lane + j)) { if (bad < 5) printf("K=%d lane=%d j=%d got %x want %x\n", K, lane, j, st[j], ring_state(w, K, 8 * lane + j)); ++bad; }
        }
    }
    return bad;
}

int main()
{
    int bad = check<1>() + check<2>() + check<3>() + check<4>() + check<5>() + check<6>() + check<7>() + check<8>();
    printf(bad ? "FAILED %d\n" : "OK %d\n", bad);
    return bad ? 1 : 0;
}
