// Exports the reference's OWN host baseline templates through a C ABI.
//
// TEST INFRASTRUCTURE. This file contains no reference code: it #includes the
// reference's op-test sources from the reference checkout at build time
// (include path given by oracle/Makefile) and instantiates their
// `baseline_*` templates. The result (oracle/_ref/libark_ref.so) is used to
// pin the C restatement in ark_oracle.c and to generate tests/golden/.
//
// Each reference test file is compiled as its own translation unit, selected
// with -DSHIM_<NAME>; the file's main() is renamed on the command line.
#include <cstdint>
#include <vector>

#if defined(SHIM_REDUCE)
#include "ops/ops_reduce_test.cpp"
#elif defined(SHIM_MATH)
#include "ops/ops_math_test.cpp"
#elif defined(SHIM_ARITH)
#include "ops/ops_arithmetic_test.cpp"
#elif defined(SHIM_ROPE)
#include "ops/ops_rope_test.cpp"
#elif defined(SHIM_CAST)
#include "ops/ops_cast_test.cpp"
#elif defined(SHIM_SCALAR)
#include "ops/ops_scalar_test.cpp"
#elif defined(SHIM_TRANSPOSE)
#include "ops/ops_transpose_test.cpp"
#elif defined(SHIM_EMBEDDING)
#include "ops/ops_embedding_test.cpp"
#elif defined(SHIM_COPY)
#include "ops/ops_copy_test.cpp"
#endif

namespace {
// Argument pack in the shape the reference's OpsTestBaseline functors take
// (ark/ops/ops_test_common.hpp:163-166).
struct Pack {
    std::vector<void *> outs, ins;
    std::vector<ark::Dims> osh, ish;
    Pack(void **o, const int64_t *os, const int *ond, int no, void **i, const int64_t *is, const int *ind,
         int ni) {
        for (int t = 0; t < no; ++t) {
            outs.push_back(o[t]);
            osh.emplace_back(std::vector<ark::DimType>(os + 4 * t, os + 4 * t + ond[t]));
        }
        for (int t = 0; t < ni; ++t) {
            ins.push_back(i[t]);
            ish.emplace_back(std::vector<ark::DimType>(is + 4 * t, is + 4 * t + ind[t]));
        }
    }
};
}  // namespace

#define REF_ARGS void **o, const int64_t *os, const int *ond, int no, void **i, const int64_t *is, const int *ind, int ni
#define REF_EXPORT(sym, ...)                                                        \
    extern "C" __attribute__((visibility("default"))) void sym(REF_ARGS) {          \
        Pack p(o, os, ond, no, i, is, ind, ni);                                     \
        __VA_ARGS__(p.outs, p.osh, p.ins, p.ish, 0);                                \
    }
#define REF_EXPORT_FLOATS(name, fn)          \
    REF_EXPORT(ref_##name##_fp32, fn<float>) \
    REF_EXPORT(ref_##name##_fp16, fn<ark::half_t>) \
    REF_EXPORT(ref_##name##_bf16, fn<ark::bfloat16_t>)

#if defined(SHIM_REDUCE)
REF_EXPORT_FLOATS(reduce_sum_axis0, baseline_reduce_sum_axis0)
REF_EXPORT_FLOATS(reduce_sum_axis1, baseline_reduce_sum_axis1)
REF_EXPORT_FLOATS(reduce_sum_axis2, baseline_reduce_sum_axis2)
REF_EXPORT_FLOATS(reduce_sum_axis3, baseline_reduce_sum_axis3)
REF_EXPORT_FLOATS(reduce_max_axis3, baseline_reduce_max_axis3)
REF_EXPORT_FLOATS(reduce_mean_axis3, baseline_reduce_mean_axis3)
#elif defined(SHIM_MATH)
REF_EXPORT_FLOATS(gelu, baseline_gelu)
REF_EXPORT_FLOATS(exp, baseline_exp)
REF_EXPORT_FLOATS(relu, baseline_relu)
REF_EXPORT_FLOATS(rsqrt, baseline_rsqrt)
REF_EXPORT_FLOATS(sigmoid, baseline_sigmoid)
REF_EXPORT_FLOATS(sqrt, baseline_sqrt)
#elif defined(SHIM_ARITH)
REF_EXPORT_FLOATS(add, baseline_add)
REF_EXPORT_FLOATS(sub, baseline_sub)
REF_EXPORT_FLOATS(mul, baseline_mul)
REF_EXPORT_FLOATS(div, baseline_div)
#elif defined(SHIM_ROPE)
REF_EXPORT_FLOATS(rope, baseline_rope)
#elif defined(SHIM_CAST)
REF_EXPORT(ref_cast_fp16_fp32, baseline_cast<ark::half_t, float>)
REF_EXPORT(ref_cast_fp32_fp16, baseline_cast<float, ark::half_t>)
REF_EXPORT(ref_cast_bf16_fp32, baseline_cast<ark::bfloat16_t, float>)
REF_EXPORT(ref_cast_fp32_bf16, baseline_cast<float, ark::bfloat16_t>)
REF_EXPORT(ref_cast_fp16_int32, baseline_cast<ark::half_t, int>)
REF_EXPORT(ref_cast_int32_fp16, baseline_cast<int, ark::half_t>)
REF_EXPORT(ref_cast_fp32_int32, baseline_cast<float, int>)
REF_EXPORT(ref_cast_int32_fp32, baseline_cast<int, float>)
#elif defined(SHIM_SCALAR)
// The reference's scalar baselines bake in the factor 0.7 (ops_scalar_test.cpp:9).
REF_EXPORT_FLOATS(scalar_add, baseline_scalar_add)
REF_EXPORT_FLOATS(scalar_sub, baseline_scalar_sub)
REF_EXPORT_FLOATS(scalar_mul, baseline_scalar_mul)
REF_EXPORT_FLOATS(scalar_div, baseline_scalar_div)
#elif defined(SHIM_TRANSPOSE)
REF_EXPORT_FLOATS(transpose_0132, baseline_transpose_0132)
REF_EXPORT_FLOATS(transpose_0231, baseline_transpose_0231)
#elif defined(SHIM_EMBEDDING)
REF_EXPORT_FLOATS(embedding, baseline_embedding)
#elif defined(SHIM_COPY)
REF_EXPORT_FLOATS(copy, baseline_copy)
#endif
