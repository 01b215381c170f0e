// Drives the C++ mirror of Qwen_Linear_with_bias_Int4 the way the reference's own
// qwen3/tests/test_linear.cc:20-66 drives the original: construct the layer from a directory
// holding the four .bin files, run forward() on an input file, write the output.
//   test_linear_mirror <dir/> <N> <K> <M> <input.bin> <output.bin>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "ink_linear.h"

int main(int argc, char **argv)
{
    if (argc != 7) return 2;
    const std::string dir = argv[1];
    const int N = std::atoi(argv[2]), K = std::atoi(argv[3]), M = std::atoi(argv[4]);
    try {
        ModelContext ctx(0);
        Qwen_Linear_with_bias_Int4 layer(&ctx, dir, 1, N, K);
        Qwen_Linear_with_bias_Int4 copy = layer;              // layers are copied into a std::vector in the reference
        Matrix3D<float> x(1, M, K);
        FILE *f = std::fopen(argv[5], "rb");
        if (!f || std::fread(x.data(), sizeof(float), x.length(), f) != x.length()) return 3;
        std::fclose(f);
        Matrix3D<float> y = copy.forward(x);
        if (y.m_dim_x != 1 || y.m_dim_y != M || y.m_dim_z != N) return 4;
        Matrix3D<float> x1(1, 1, K);                             // decode path: m == 1
        for (int k = 0; k < K; k++) x1(0, 0, k) = x(0, 0, k);
        Matrix3D<float> y1 = layer.forward(x1);
        f = std::fopen(argv[6], "wb");
        std::fwrite(y.data(), sizeof(float), y.length(), f);
        std::fwrite(y1.data(), sizeof(float), y1.length(), f);
        std::fclose(f);
        bool threw = false;                                      // a missing file raises, as read_to_array does
        try {
            Qwen_Linear_with_bias_Int4 bad(&ctx, dir + "missing/", 1, N, K);
        } catch (const std::runtime_error &) {
            threw = true;
        }
        return threw ? 0 : 5;
    } catch (const std::exception &e) {
        std::fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
}
