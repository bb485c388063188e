/*
 * C entry points over the reference's OWN CPU helpers for the dequantise + matmul path.
 *
 * TEST INFRASTRUCTURE ONLY (as everything under oracle/): used to validate the restatement in
 * dequant_oracle.c and as the timed CPU baseline.  Nothing in the shipped package links it.
 *
 * The helpers are member functions of the reference's GoogleTest fixture,
 * tests/cpp/test_dequant_matmul.mm:103-259 (pack_int4, dequant_reference_int4,
 * dequant_reference_int8, matmul_reference, fp16_to_fp32, fp32_to_fp16).  The file as a whole
 * needs Objective-C++, Metal headers and GoogleTest, but those lines are plain C++ that touch
 * none of it.  build_ref.py copies exactly that line range, unmodified, out of the reference
 * checkout into _ref/ref_helpers.inc (a build product, never committed) and this file includes
 * it as the body of a struct, so the code that runs is the reference's own text.
 */
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

namespace {
struct RefHelpers {
#include "_ref/ref_helpers.inc"
};
}  // namespace

extern "C" {

void ref_pack_int4(const int8_t* values, size_t n, uint8_t* out)
{
    RefHelpers h;
    const std::vector<uint8_t> p = h.pack_int4(std::vector<int8_t>(values, values + n));
    std::memcpy(out, p.data(), p.size());
}

float ref_fp16_to_fp32(uint16_t v) { return RefHelpers::fp16_to_fp32(v); }
uint16_t ref_fp32_to_fp16(float v) { return RefHelpers::fp32_to_fp16(v); }

void ref_dequant_int4(const uint8_t* packed, const float* scales, const float* zeros, uint32_t K, uint32_t N,
                      uint32_t group_size, float* out)
{
    RefHelpers h;
    const uint32_t G = (K + group_size - 1) / group_size;
    const std::vector<float> w = h.dequant_reference_int4(
        std::vector<uint8_t>(packed, packed + (size_t)N * ((K + 1) / 2)), std::vector<float>(scales, scales + (size_t)N * G),
        std::vector<float>(zeros, zeros + (size_t)N * G), K, N, group_size);
    std::memcpy(out, w.data(), w.size() * sizeof(float));
}

void ref_dequant_int8(const int8_t* data, const float* scales, const float* zeros, uint32_t K, uint32_t N,
                      uint32_t group_size, float* out)
{
    RefHelpers h;
    const uint32_t G = (K + group_size - 1) / group_size;
    const std::vector<float> w = h.dequant_reference_int8(
        std::vector<int8_t>(data, data + (size_t)N * K), std::vector<float>(scales, scales + (size_t)N * G),
        std::vector<float>(zeros, zeros + (size_t)N * G), K, N, group_size);
    std::memcpy(out, w.data(), w.size() * sizeof(float));
}

void ref_matmul(const float* A, const float* B, uint32_t M, uint32_t N, uint32_t K, float* C)
{
    RefHelpers h;
    const std::vector<float> c = h.matmul_reference(std::vector<float>(A, A + (size_t)M * K),
                                                    std::vector<float>(B, B + (size_t)N * K), M, N, K);
    std::memcpy(C, c.data(), c.size() * sizeof(float));
}

/* The reference's whole CPU path for rows [n_begin, n_end) of the weight matrix: dequantise them to
 * fp32, then the naive matmul; C is [M, n_end - n_begin].  quant: 0 = int4, 1 = int8.  The caller
 * may run several row ranges on several threads (the helpers keep no state). */
void ref_dequant_matmul_rows(const float* A, const void* wq, const float* scales, const float* zeros, uint32_t M,
                             uint32_t K, uint32_t group_size, int quant, uint32_t n_begin, uint32_t n_end, float* C)
{
    RefHelpers h;
    const uint32_t G = (K + group_size - 1) / group_size;
    const uint32_t n = n_end - n_begin;
    const std::vector<float> s(scales + (size_t)n_begin * G, scales + (size_t)n_end * G);
    const std::vector<float> z(zeros + (size_t)n_begin * G, zeros + (size_t)n_end * G);
    std::vector<float> w;
    if (quant == 0) {
        const size_t rb = (K + 1) / 2;
        const uint8_t* p = static_cast<const uint8_t*>(wq);
        w = h.dequant_reference_int4(std::vector<uint8_t>(p + n_begin * rb, p + n_end * rb), s, z, K, n, group_size);
    } else {
        const int8_t* p = static_cast<const int8_t*>(wq);
        w = h.dequant_reference_int8(std::vector<int8_t>(p + (size_t)n_begin * K, p + (size_t)n_end * K), s, z, K, n,
                                     group_size);
    }
    const std::vector<float> c = h.matmul_reference(std::vector<float>(A, A + (size_t)M * K), w, M, n, K);
    std::memcpy(C, c.data(), c.size() * sizeof(float));
}

}  // extern "C"
