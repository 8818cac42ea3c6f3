// Driver around the reference's own src/layers/embed.h (included from the
// reference tree at build time, never copied): prints sinusoidal_time_emb(t, dim,
// min_p, max_p) as hex floats so golden vectors carry every bit.
// usage: time_emb_ref <t> <dim> <min_p> <max_p>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cstdint>
#include <limits>
#include <vector>
#include "layers/embed.h"

int main(int argc, char **argv) {
    if (argc != 5) return 2;
    const double t = std::atof(argv[1]);
    const long dim = std::atol(argv[2]);
    const double mn = std::atof(argv[3]), mx = std::atof(argv[4]);
    const std::vector<float> v = vla::sinusoidal_time_emb(t, dim, mn, mx);
    for (float f : v) {
        uint32_t u;
        std::memcpy(&u, &f, 4);
        std::printf("%08x\n", u);
    }
    return 0;
}
