// TEST INFRASTRUCTURE ONLY.  Drives the REFERENCE's own linear-layer class, compiled unmodified from a checkout of
// the reference project (oracle/Makefile, target `dropin`): constructs ModelContext and Qwen_Linear_with_bias_Int4
// from a layer directory holding the four .bin files the reference exports
// (qwen3/include/qwen/QwenOperator.h:112-157) and calls its forward (qwen3/src/qwen/QwenOperator.cc:80-124).
// The same driver is linked twice:
//   ref_linear_cpu      with the reference's own CPU kernels (quantized_gemx_kernels.cc)
//   ref_linear_on_gpu   WITHOUT that file, against libinkq_refshim.so: the reference-named functions of this
//                       repository, running on the GPU
// so that a test can show the reference's class producing the same result on either.
//
//   ref_linear_* <layer dir with trailing slash> <N> <K> <M> <x.bin: fp32 [M][K]> <out.bin: fp32 [M][N]>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "QwenOperator.h"

int main(int argc, char **argv)
{
    if (argc != 7) {
        fprintf(stderr, "usage: %s layer_dir/ N K M x.bin out.bin\n", argv[0]);
        return 2;
    }
    const std::string dir = argv[1];
    const int N = atoi(argv[2]), K = atoi(argv[3]), M = atoi(argv[4]);
    ModelContext ctx;
    // staging for the four files, as QwenForCausalLM.cc:87-99 sizes it for its largest layer
    const size_t wbytes = static_cast<size_t>(N) * K / 2 + 2 * sizeof(float) * (static_cast<size_t>(N) * K / 32) + static_cast<size_t>(N) * K / 32;
    ctx.repack_buffer = make_aligned_x86<int8_t>(64, wbytes + 64);
    // quantized activations; six rows of padding because the reference's GEMM reads up to five rows past M
    // (quantized_gemx_kernels.cc:371-375)
    const size_t abytes = sizeof(q8_repack_1x2_fp32) * (static_cast<size_t>(M) + 6) * (K / 64);
    ctx.activation_buffer = make_aligned_x86<int8_t>(64, abytes);
    for (size_t i = 0; i < abytes; i++) ctx.activation_buffer.get()[i] = 0;
    try {
        Qwen_Linear_with_bias_Int4 layer(&ctx, dir, 1, N, K);
        std::vector<float> xin(static_cast<size_t>(M) * K);
        FILE *f = fopen(argv[5], "rb");
        if (f == nullptr || fread(xin.data(), sizeof(float), xin.size(), f) != xin.size()) {
            fprintf(stderr, "cannot read %s\n", argv[5]);
            return 3;
        }
        fclose(f);
        Matrix3D<float> x(xin.data(), 1, M, K);
        Matrix3D<float> y = layer.forward(x);
        f = fopen(argv[6], "wb");
        if (f == nullptr || fwrite(y.data(), sizeof(float), static_cast<size_t>(M) * N, f) != static_cast<size_t>(M) * N) {
            fprintf(stderr, "cannot write %s\n", argv[6]);
            return 4;
        }
        fclose(f);
    } catch (const std::exception &e) {
        fprintf(stderr, "error: %s\n", e.what());
        return 5;
    }
    return 0;
}
