// Host-side C++ mirror of the reference's quantized linear layer, on top of the C ABI.
//
// Same names, constructor arguments, forward() signature and error behaviour as
// Qwen_Linear_with_bias_Int4 (qwen3/include/qwen/QwenOperator.h:86-231,
// qwen3/src/qwen/QwenOperator.cc:80-124), for a host that owns such layers the way the
// reference's model code does (QwenAttention.cc:29-30, QwenDecoderLayer.cc:21-23,
// QwenForCausalLM.cc:121).  The weights live on the GPU; forward() copies the activations
// in and the result out (inkq_linear_host).  It is a stand-alone class, not a replacement
// header for the reference tree: the reference's own class and ModelContext (which also
// carries the KV caches and the CPU staging buffers) run on the GPU unchanged when the
// reference's QwenOperator.cc is linked against libinkq_refshim.so (ref_names.cc) instead
// of its quantized_gemx_kernels.cc.
//
// When this header is used inside the reference tree, define INK_USE_REFERENCE_COMMON
// before including it so that the reference's own Matrix3D (qwen3/include/common.h) is
// used instead of the minimal stand-in below.
#pragma once
#include <cstdint>
#include <cstdio>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "inkq.h"

#ifndef QK
#define QK 32  // quantization block (qwen3/include/qwen/QwenConfig.h:8)
#endif

#ifndef INK_USE_REFERENCE_COMMON
// The part of the reference's Matrix3D contract the linear layer relies on
// (qwen3/include/common.h:13-364): owning, row-major x*y*z, public dims, data().
template <typename T>
class Matrix3D {
   public:
    Matrix3D() : m_dim_x(0), m_dim_y(0), m_dim_z(0) {}
    Matrix3D(int x, int y, int z) : m_dim_x(x), m_dim_y(y), m_dim_z(z), m_data(new T[static_cast<size_t>(x) * y * z]()) {}
    T *data() const { return m_data.get(); }
    T &operator()(int x, int y, int z) { return m_data[(static_cast<size_t>(x) * m_dim_y + y) * m_dim_z + z]; }
    const T &operator()(int x, int y, int z) const { return m_data[(static_cast<size_t>(x) * m_dim_y + y) * m_dim_z + z]; }
    size_t length() const { return static_cast<size_t>(m_dim_x) * m_dim_y * m_dim_z; }
    int m_dim_x, m_dim_y, m_dim_z;

   private:
    std::unique_ptr<T[]> m_data;
};
#endif

// The part of the reference's ModelContext (QwenOperator.h:34-43) this class needs: the
// reference's CPU staging and activation scratch are replaced by the device context, which
// owns the activation scratch on the GPU; the KV caches belong to the attention operator
// and have no place here.
struct ModelContext {
    inkq_ctx *gpu = nullptr;
    explicit ModelContext(int device = 0)
    {
        if (inkq_ctx_create(device, nullptr, &gpu) != INKQ_OK) throw std::runtime_error(std::string("inkq: ") + inkq_last_error(nullptr));
    }
    ~ModelContext() { inkq_ctx_destroy(gpu); }
    ModelContext(const ModelContext &) = delete;
    ModelContext &operator=(const ModelContext &) = delete;
};

namespace ink_detail {
// read_to_array of the reference (qwen3/src/utils.cc:12-28): whole file into a buffer, exception on failure
template <typename T>
inline void read_file(const std::string &path, std::vector<T> &out, size_t count)
{
    out.resize(count);
    FILE *f = std::fopen(path.c_str(), "rb");
    if (f == nullptr) throw std::runtime_error("failed to open file: " + path);
    const size_t got = std::fread(out.data(), sizeof(T), count, f);
    std::fclose(f);
    if (got != count) throw std::runtime_error("failed to read file: " + path);
}
struct WeightDeleter {
    void operator()(inkq_weight *w) const { inkq_weight_destroy(w); }
};
}  // namespace ink_detail

class Qwen_Linear_with_bias_Int4 {
    int weight_cols = 0, weight_rows = 0;  // N, K as in the reference (QwenOperator.h:95,143-144)
    bool has_bias = false;
    ModelContext *context_ = nullptr;
    // Copies of a layer share the (immutable) device weights; the reference deep-copies its CPU
    // buffers because its layers live in a std::vector (QwenOperator.h:160-222) - same semantics.
    std::shared_ptr<inkq_weight> weight_;

   public:
    Qwen_Linear_with_bias_Int4() = default;

    // path holds weight_int4.bin, scaling_factor_int4.bin, offset_int4.bin, zero_point_int4.bin
    // (QwenOperator.h:137-140); weight_dim_x must be 1, weight_dim_y = N, weight_dim_z = K.
    Qwen_Linear_with_bias_Int4(ModelContext *ctx, std::string path, int weight_dim_x, int weight_dim_y, int weight_dim_z)
        : weight_cols(weight_dim_y), weight_rows(weight_dim_z), context_(ctx)
    {
        if (weight_dim_x != 1) throw std::invalid_argument("weight_dim_x must be 1");
        const size_t N = weight_dim_y, K = weight_dim_z;
        std::vector<uint8_t> q4;
        std::vector<float> scale, offset;
        ink_detail::read_file(path + "weight_int4.bin", q4, N * K / 2);
        ink_detail::read_file(path + "scaling_factor_int4.bin", scale, N * K / QK);
        ink_detail::read_file(path + "offset_int4.bin", offset, N * K / QK);
        // zero_point_int4.bin is loaded but never used by the reference's kernels (QwenOperator.h:140): not needed here
        init(q4.data(), scale.data(), offset.data());
    }

    // Same layer from tensors already in memory (logical on-disk format).
    Qwen_Linear_with_bias_Int4(ModelContext *ctx, int N, int K, const uint8_t *weight_int4, const float *scaling_factor, const float *offset)
        : weight_cols(N), weight_rows(K), context_(ctx)
    {
        init(weight_int4, scaling_factor, offset);
    }

    // m = activation.m_dim_y rows, k = activation.m_dim_z; returns a fresh (bs, m, n) matrix
    // (QwenOperator.cc:80-124).  m > 1 takes the QGEMM, m == 1 the QGEMV, as in the reference.
    Matrix3D<float> forward(const Matrix3D<float> &activation)
    {
        const int bs = activation.m_dim_x, m = activation.m_dim_y, n = weight_cols, k = activation.m_dim_z;
        if (bs != 1 || k != weight_rows) throw std::invalid_argument("activation shape does not match the layer");
        Matrix3D<float> output(bs, m, n);
        if (inkq_linear_host(context_->gpu, weight_.get(), activation.data(), m, output.data(), n) != INKQ_OK)
            throw std::runtime_error(std::string("inkq: ") + inkq_last_error(context_->gpu));
        return output;
    }

    int cols() const { return weight_cols; }
    int rows() const { return weight_rows; }

   private:
    void init(const uint8_t *q4, const float *scale, const float *offset)
    {
        inkq_weight *w = nullptr;
        if (inkq_weight_create(context_->gpu, INKQ_A81W41, INKQ_SCALES_F32, weight_cols, weight_rows, q4, scale, offset, nullptr, 0, weight_cols,
                               &w) != INKQ_OK)
            throw std::runtime_error(std::string("inkq: ") + inkq_last_error(context_->gpu));
        weight_ = std::shared_ptr<inkq_weight>(w, ink_detail::WeightDeleter());
    }
};
