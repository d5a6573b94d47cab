// The CUDA provider: selects a hand-written sm_100a kernel for a typed tcrv_rvv body by op
// identity and typed facts, validates the selected lowering boundary fail-closed, realizes
// pre-realized bodies, and builds the emission plan that names the C-ABI launcher.
//
// Behaviour mirrored from the reference's RVV provider: readiness -> plan -> boundary
// materialisation (lib/Plugin/RVV/RVVExtensionPlugin.cpp:536-712), pre-realized body
// realization (lib/Plugin/RVV/RVVSelectedBodyRealization.cpp:214-244), and the pinned
// block-format facts of the quantized ops (lib/Dialect/RVV/IR/RVVDialectWideningOps.cpp:993-1183).
#include "tcrv/CUDAPlugin.h"

#include <sstream>

namespace tcrv {
namespace cuda {

const char *const kPluginName = "cuda-plugin";
const char *const kCapabilityId = "cuda.sm_100a";
const char *const kCapabilityKind = "accelerator";
const char *const kProtocolAttr = "cuda_construction_protocol";
const char *const kProtocolValue = "extension-family-construction-protocol.v1";
const char *const kRouteId = "cuda-sm100a-typed-body-launch-route-family";
const char *const kEmissionKind = "prebuilt-sm100a-kernel-c-abi-launch";
const char *const kArtifactKind = "cuda-sm100a-launch-descriptor";
const char *const kBoundaryOp = "tcrv_rvv.with_vl";
const char *const kRuntimeABIKind = "plugin-owned-runtime-abi";
const char *const kGlueRole = "cuda-c-abi-launch-runtime-glue";

namespace {

using Sig = std::vector<std::pair<std::string, std::string>>;  // (role, c_type) in ABI order

const std::vector<Fact> kQ4Q8Facts = {
    {"scale_model", false, "dual-fp16-per-block-d_x.d_y", 0}, {"qk", true, "", 32},
    {"weight_block_stride", true, "", 18},                    {"activation_block_stride", true, "", 34},
    {"quant_byte_offset", true, "", 2},                       {"activation_high_byte_offset", true, "", 16}};

const std::vector<Fact> kQ8Q8Facts = {{"scale_model", false, "dual-fp16-per-block-d_x.d_y", 0},
                                      {"qk", true, "", 32},
                                      {"weight_block_stride", true, "", 34},
                                      {"activation_block_stride", true, "", 34},
                                      {"quant_byte_offset", true, "", 2}};

std::vector<Fact> withKind(const char *kind, std::vector<Fact> rest) {
  rest.insert(rest.begin(), Fact{"kind", false, kind, 0});
  return rest;
}

std::vector<RouteEntry> buildTable() {
  std::vector<RouteEntry> t;
  const Sig addF32 = {{"lhs-input-buffer", "const float *"},
                      {"rhs-input-buffer", "const float *"},
                      {"output-buffer", "float *"},
                      {"runtime-element-count", "size_t"}};
  const Sig addI32 = {{"lhs-input-buffer", "const int32_t *"},
                      {"rhs-input-buffer", "const int32_t *"},
                      {"output-buffer", "int32_t *"},
                      {"runtime-element-count", "size_t"}};
  t.push_back({"tcrv_rvv.binary", withKind("add", {}), "f32", {"tcrv_rvv.load", "tcrv_rvv.load", "tcrv_rvv.binary", "tcrv_rvv.store"},
               {}, addF32, "add", "cuda-generic-binary-add-f32-callable-c-abi.v1", "tcrv_cuda_add_f32",
               "tcrv_cuda_host_add_f32", "streaming-elementwise", "hbm", ""});
  t.push_back({"tcrv_rvv.binary", withKind("add", {}), "i32", {"tcrv_rvv.load", "tcrv_rvv.load", "tcrv_rvv.binary", "tcrv_rvv.store"},
               {}, addI32, "add", "cuda-generic-binary-add-i32-callable-c-abi.v1", "tcrv_cuda_add_i32",
               "tcrv_cuda_host_add_i32", "streaming-elementwise", "hbm", ""});
  t.push_back({"tcrv_rvv.dequantize",
               withKind("i32_to_f32_scaled", {{"dequant_relation", false, "signed-i32m1-to-f32m1-scale-f32", 0}}), "",
               {"tcrv_rvv.load", "tcrv_rvv.dequantize", "tcrv_rvv.store"}, {},
               {{"lhs-input-buffer", "const int32_t *"}, {"dequant-scale-value", "float"}, {"output-buffer", "float *"},
                {"runtime-element-count", "size_t"}},
               "dequantize_i32_to_f32", "cuda-generic-dequantize-i32-f32-callable-c-abi.v1",
               "tcrv_cuda_dequantize_i32_f32", "tcrv_cuda_host_dequantize_i32_f32", "streaming-elementwise", "hbm", ""});
  t.push_back({"tcrv_rvv.quantize_row_q8_0",
               withKind("ggml_quantize_row_q8_0", {{"qk", true, "", 32}, {"block_stride", true, "", 34},
                                                   {"scale_byte_offset", true, "", 0}, {"quant_byte_offset", true, "", 2}}),
               "", {"tcrv_rvv.quantize_row_q8_0"},
               {"lhs-input-buffer", "output-buffer", "runtime-element-count"},
               {{"runtime-element-count", "size_t"}, {"lhs-input-buffer", "const float *"}, {"output-buffer", "uint8_t *"}},
               "quantize_row_q8_0", "cuda-ggml-quantize-row-q8_0-callable-c-abi.v1", "tcrv_cuda_quantize_row_q8_0",
               "tcrv_cuda_host_quantize_row_q8_0", "streaming-quantizer", "hbm", ""});
  // sibling block formats (general strict-order kernel)
  {
    const Sig dotSig = {{"runtime-element-count", "size_t"}, {"output-buffer", "float *"},
                        {"lhs-input-buffer", "const uint8_t *"}, {"rhs-input-buffer", "const uint8_t *"}};
    const std::vector<std::string> dotRoles = {"lhs-input-buffer", "rhs-input-buffer", "output-buffer",
                                               "runtime-element-count"};
    t.push_back({"tcrv_rvv.q4_1_q8_1_block_dot",
                 withKind("ggml_q4_1_q8_1_block_dot",
                          {{"scale_model", false, "dual-fp16-per-block-d_x.d_y-plus-min", 0}, {"qk", true, "", 32},
                           {"weight_block_stride", true, "", 20}, {"activation_block_stride", true, "", 36},
                           {"quant_byte_offset", true, "", 4}, {"activation_high_byte_offset", true, "", 16},
                           {"weight_min_byte_offset", true, "", 2}, {"activation_sum_byte_offset", true, "", 2}}),
                 "", {"tcrv_rvv.q4_1_q8_1_block_dot"}, dotRoles, dotSig, "q4_1_q8_1_block_dot",
                 "cuda-ggml-q4_1-q8_1-block-dot-callable-c-abi.v1", "tcrv_cuda_vec_dot_q4_1_q8_1",
                 "tcrv_cuda_host_vec_dot_q4_1_q8_1", "block-dot-strict-order", "hbm",
                 "sumf = sumf + fma(d_x*d_y, (float)sumi, m_x*s_y), ascending blocks"});
    t.push_back({"tcrv_rvv.q5_0_q8_0_block_dot",
                 withKind("ggml_q5_0_q8_0_block_dot",
                          {{"scale_model", false, "dual-fp16-per-block-d_x.d_y", 0}, {"qk", true, "", 32},
                           {"weight_block_stride", true, "", 22}, {"activation_block_stride", true, "", 34},
                           {"quant_byte_offset", true, "", 6}, {"activation_quant_byte_offset", true, "", 2},
                           {"activation_high_byte_offset", true, "", 16}, {"weight_qh_byte_offset", true, "", 2}}),
                 "", {"tcrv_rvv.q5_0_q8_0_block_dot"}, dotRoles, dotSig, "q5_0_q8_0_block_dot",
                 "cuda-ggml-q5_0-q8_0-block-dot-callable-c-abi.v1", "tcrv_cuda_vec_dot_q5_0_q8_0",
                 "tcrv_cuda_host_vec_dot_q5_0_q8_0", "block-dot-strict-order", "hbm",
                 "sumf = fma(d_x*d_y, (float)sumi, sumf), ascending blocks"});
    t.push_back({"tcrv_rvv.q5_1_q8_1_block_dot",
                 withKind("ggml_q5_1_q8_1_block_dot",
                          {{"scale_model", false, "dual-fp16-per-block-d_x.d_y-plus-min", 0}, {"qk", true, "", 32},
                           {"weight_block_stride", true, "", 24}, {"activation_block_stride", true, "", 36},
                           {"quant_byte_offset", true, "", 8}, {"activation_quant_byte_offset", true, "", 4},
                           {"activation_high_byte_offset", true, "", 16}, {"weight_qh_byte_offset", true, "", 4},
                           {"weight_min_byte_offset", true, "", 2}, {"activation_sum_byte_offset", true, "", 2}}),
                 "", {"tcrv_rvv.q5_1_q8_1_block_dot"}, dotRoles, dotSig, "q5_1_q8_1_block_dot",
                 "cuda-ggml-q5_1-q8_1-block-dot-callable-c-abi.v1", "tcrv_cuda_vec_dot_q5_1_q8_1",
                 "tcrv_cuda_host_vec_dot_q5_1_q8_1", "block-dot-strict-order", "hbm",
                 "sumf = sumf + fma(d_x*d_y, (float)sumi, m_x*s_y), ascending blocks"});
  }
  // weight repack into the reference's 16-row interleaved layout
  t.push_back({"tcrv_rvv.pack_q4_0_to_q4_0x16",
               withKind("ggml_pack_q4_0_to_q4_0x16",
                        {{"qk", true, "", 32}, {"src_block_stride", true, "", 18}, {"dst_block_stride", true, "", 288},
                         {"src_quant_byte_offset", true, "", 2}, {"dst_quant_byte_offset", true, "", 32},
                         {"weight_interleave", true, "", 16}, {"xor_mask", true, "", 136}}),
               "", {"tcrv_rvv.pack_q4_0_to_q4_0x16"},
               {"lhs-input-buffer", "output-buffer", "runtime-element-count"},
               {{"runtime-element-count", "size_t"}, {"lhs-input-buffer", "const uint8_t *"},
                {"output-buffer", "uint8_t *"}},
               "pack_q4_0_to_q4_0x16", "cuda-ggml-pack-q4_0-to-q4_0x16-callable-c-abi.v1",
               "tcrv_cuda_pack_q4_0_to_q4_0x16", "tcrv_cuda_host_pack_q4_0_to_q4_0x16", "streaming-byte-permutation",
               "hbm", ""});
  // consumers of the interleaved layouts (lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:2122, 2853, 3930)
  {
    const std::vector<std::string> gemvRoles = {"lhs-input-buffer", "rhs-input-buffer", "output-buffer",
                                                "runtime-element-count", "destination-byte-stride"};
    const std::vector<std::pair<std::string, std::string>> gemvSig = {
        {"runtime-element-count", "size_t"}, {"output-buffer", "float *"}, {"lhs-input-buffer", "const uint8_t *"},
        {"rhs-input-buffer", "const uint8_t *"}, {"destination-byte-stride", "size_t"}};
    t.push_back({"tcrv_rvv.repack_gemv_q4_0_q8_0",
                 withKind("ggml_repack_gemv_q4_0_q8_0",
                          {{"scale_model", false, "dual-fp16-per-block-d_x.d_y", 0}, {"qk", true, "", 32},
                           {"weight_block_stride", true, "", 288}, {"activation_block_stride", true, "", 34},
                           {"weight_quant_byte_offset", true, "", 32}, {"activation_quant_byte_offset", true, "", 2},
                           {"weight_interleave", true, "", 16}}),
                 "", {"tcrv_rvv.repack_gemv_q4_0_q8_0"}, gemvRoles, gemvSig, "repack_gemv_q4_0_q8_0",
                 "cuda-ggml-repack-gemv-q4_0-q8_0-callable-c-abi.v1", "tcrv_cuda_repack_gemv_q4_0_q8_0",
                 "tcrv_cuda_host_repack_gemv_q4_0_q8_0", "decode-gemv-x16-bulk-copy", "hbm",
                 "fma((float)sumi, d_w*d_a, .); host entry: strict ascending blocks (the reference's lane-wise chain); "
                 "device entry without TCRV_CUDA_FLAG_STRICT_ORDER: 8 interleaved chains per range, ranges ascending"});
    t.back().layoutNote =
        "compatibility path: the 16-row interleaved layout is made for RVV lanes; on sm_100a plain block rows are the "
        "native layout (streaming GEMV 12.6 us against 16.5 us here for 32000x4096), so repack only when the caller "
        "already holds x16 weights";
    t.push_back({"tcrv_rvv.repack_gemv_q8_0_q8_0",
                 withKind("ggml_repack_gemv_q8_0_q8_0",
                          {{"scale_model", false, "dual-fp16-per-block-d_x.d_y", 0}, {"qk", true, "", 32},
                           {"weight_block_stride", true, "", 544}, {"activation_block_stride", true, "", 34},
                           {"weight_quant_byte_offset", true, "", 32}, {"activation_quant_byte_offset", true, "", 2},
                           {"weight_interleave", true, "", 16}}),
                 "", {"tcrv_rvv.repack_gemv_q8_0_q8_0"}, gemvRoles, gemvSig, "repack_gemv_q8_0_q8_0",
                 "cuda-ggml-repack-gemv-q8_0-q8_0-callable-c-abi.v1", "tcrv_cuda_repack_gemv_q8_0_q8_0",
                 "tcrv_cuda_host_repack_gemv_q8_0_q8_0", "decode-gemv-x16-bulk-copy", "hbm",
                 "fma((float)sumi, d_w*d_a, .); host entry: strict ascending blocks (the reference's lane-wise chain); "
                 "device entry without TCRV_CUDA_FLAG_STRICT_ORDER: 8 interleaved chains per range, ranges ascending"});
    t.back().layoutNote =
        "compatibility path: the 16-row interleaved layout is made for RVV lanes; on sm_100a plain block rows are the "
        "native layout (streaming GEMV 12.6 us against 16.5 us here for 32000x4096), so repack only when the caller "
        "already holds x16 weights";
    t.push_back({"tcrv_rvv.repack_gemm_q4_0_q8_0",
                 withKind("ggml_repack_gemm_q4_0_q8_0",
                          {{"scale_model", false, "dual-fp16-per-block-d_x.d_y", 0}, {"qk", true, "", 32},
                           {"weight_block_stride", true, "", 288}, {"activation_block_stride", true, "", 136},
                           {"weight_quant_byte_offset", true, "", 32}, {"activation_quant_byte_offset", true, "", 8},
                           {"weight_interleave", true, "", 16}, {"activation_interleave", true, "", 4}}),
                 "", {"tcrv_rvv.repack_gemm_q4_0_q8_0"},
                 {"lhs-input-buffer", "rhs-input-buffer", "output-buffer", "runtime-element-count",
                  "source-byte-stride", "destination-byte-stride", "output-stride"},
                 {{"runtime-element-count", "size_t"}, {"output-buffer", "float *"},
                  {"lhs-input-buffer", "const uint8_t *"}, {"rhs-input-buffer", "const uint8_t *"},
                  {"source-byte-stride", "size_t"}, {"destination-byte-stride", "size_t"}, {"output-stride", "size_t"}},
                 "repack_gemm_q4_0_q8_0", "cuda-ggml-repack-gemm-q4_0-q8_0-callable-c-abi.v1",
                 "tcrv_cuda_repack_gemm_q4_0_q8_0", "tcrv_cuda_host_repack_gemm_q4_0_q8_0",
                 "prefill-gemm-tcgen05-i8-token-major", "tensor",
                 "fma((float)sumi, d_w*d_a, .), ascending blocks per element"});
  }
  // f32 forward-pass ops around the matmul (lib/Conversion/RVV/RVVToEmitCForwardElementwise.cpp)
  t.push_back({"tcrv_rvv.ggml_vec_scale_f32", withKind("ggml_vec_scale_f32", {}), "", {"tcrv_rvv.ggml_vec_scale_f32"},
               {"output-buffer", "dequant-scale-value", "runtime-element-count"},
               {{"runtime-element-count", "size_t"}, {"output-buffer", "float *"}, {"dequant-scale-value", "float"}},
               "ggml_vec_scale_f32", "cuda-ggml-vec-scale-f32-callable-c-abi.v1", "tcrv_cuda_vec_scale_f32",
               "tcrv_cuda_host_vec_scale_f32", "streaming-elementwise", "hbm", ""});
  t.push_back({"tcrv_rvv.ggml_rms_norm_f32", withKind("ggml_rms_norm_f32", {}), "", {"tcrv_rvv.ggml_rms_norm_f32"},
               {"lhs-input-buffer", "output-buffer", "dequant-scale-value", "runtime-element-count"},
               {{"runtime-element-count", "size_t"}, {"lhs-input-buffer", "const float *"}, {"output-buffer", "float *"},
                {"dequant-scale-value", "float"}},
               "ggml_rms_norm_f32", "cuda-ggml-rms-norm-f32-callable-c-abi.v1", "tcrv_cuda_rms_norm_f32",
               "tcrv_cuda_host_rms_norm_f32", "row-reduction-f64-then-scale", "hbm", ""});
  t.push_back({"tcrv_rvv.ggml_vec_silu_f32", withKind("ggml_vec_silu_f32", {}), "", {"tcrv_rvv.ggml_vec_silu_f32"},
               {"lhs-input-buffer", "output-buffer", "runtime-element-count"},
               {{"runtime-element-count", "size_t"}, {"lhs-input-buffer", "const float *"}, {"output-buffer", "float *"}},
               "ggml_vec_silu_f32", "cuda-ggml-vec-silu-f32-callable-c-abi.v1", "tcrv_cuda_vec_silu_f32",
               "tcrv_cuda_host_vec_silu_f32", "streaming-elementwise-exp-polynomial", "hbm", ""});
  {
    RouteEntry e{"tcrv_rvv.ggml_vec_soft_max_f32", withKind("ggml_vec_soft_max_f32", {}), "",
                 {"tcrv_rvv.ggml_vec_soft_max_f32"},
                 {"output-buffer", "lhs-input-buffer", "dequant-scale-value", "runtime-element-count"},
                 {{"runtime-element-count", "size_t"}, {"output-buffer", "float *"}, {"lhs-input-buffer", "const float *"},
                  {"dequant-scale-value", "float"}},
                 "ggml_vec_soft_max_f32", "cuda-ggml-vec-soft-max-f32-callable-c-abi.v1", "tcrv_cuda_vec_soft_max_f32",
                 "tcrv_cuda_host_vec_soft_max_f32", "streaming-elementwise-exp-polynomial+f64-sum", "hbm", ""};
    e.returnType = "double";
    t.push_back(e);
  }
  t.push_back({"tcrv_rvv.ggml_rope_norm_f32", withKind("ggml_rope_norm_f32", {}), "", {"tcrv_rvv.ggml_rope_norm_f32"},
               {"lhs-input-buffer", "output-buffer", "dequant-scale-value", "dequant-scale-value",
                "runtime-element-count"},
               {{"runtime-element-count", "size_t"}, {"lhs-input-buffer", "const float *"}, {"output-buffer", "float *"},
                {"dequant-scale-value", "float"}, {"dequant-scale-value", "float"}},
               "ggml_rope_norm_f32", "cuda-ggml-rope-norm-f32-callable-c-abi.v1",
               "tcrv_cuda_rope_cache_f32|tcrv_cuda_rope_apply_f32", "tcrv_cuda_host_rope_norm_f32",
               "angle-cache+pair-rotation", "hbm", ""});
  t.push_back({"tcrv_rvv.q4_0_q8_0_block_dot", withKind("ggml_q4_0_q8_0_block_dot", kQ4Q8Facts), "",
               {"tcrv_rvv.q4_0_q8_0_block_dot"},
               {"lhs-input-buffer", "rhs-input-buffer", "output-buffer", "runtime-element-count"},
               {{"runtime-element-count", "size_t"}, {"output-buffer", "float *"}, {"output-stride", "size_t"},
                {"lhs-input-buffer", "const uint8_t *"}, {"lhs-input-stride", "size_t"},
                {"rhs-input-buffer", "const uint8_t *"}, {"rhs-input-stride", "size_t"},
                {"rhs-scalar-value", "int32_t"}},
               "q4_0_q8_0_block_dot", "cuda-ggml-q4_0-q8_0-block-dot-callable-c-abi.v1", "tcrv_cuda_vec_dot_q4_0_q8_0",
               "tcrv_emitc_ggml_vec_dot_q4_0_q8_0_kernel_ggml_vec_dot_q4_0_q8_0", "block-dot-strict-order", "hbm",
               "sumf = fma((float)sumi * d_x, d_y, sumf), ascending blocks"});
  t.push_back({"tcrv_rvv.q8_0_q8_0_block_dot", withKind("ggml_q8_0_q8_0_block_dot", kQ8Q8Facts), "",
               {"tcrv_rvv.q8_0_q8_0_block_dot"},
               {"lhs-input-buffer", "rhs-input-buffer", "output-buffer", "runtime-element-count"},
               {{"runtime-element-count", "size_t"}, {"output-buffer", "float *"},
                {"lhs-input-buffer", "const uint8_t *"}, {"rhs-input-buffer", "const uint8_t *"}},
               "q8_0_q8_0_block_dot", "cuda-ggml-q8_0-q8_0-block-dot-callable-c-abi.v1", "tcrv_cuda_vec_dot_q8_0_q8_0",
               "tcrv_emitc_ggml_vec_dot_q8_0_q8_0_kernel_ggml_vec_dot_q8_0_q8_0", "block-dot-strict-order", "hbm",
               "sumf = fma((float)sumi, d_x * d_y, sumf), ascending blocks"});
  t.push_back({"tcrv_rvv.q4_0_q8_0_gemm", withKind("ggml_q4_0_q8_0_gemm", kQ4Q8Facts), "",
               {"tcrv_rvv.q4_0_q8_0_gemm"},
               {"lhs-input-buffer", "rhs-input-buffer", "rhs-input-stride", "output-buffer", "runtime-element-count",
                "source-byte-stride", "destination-byte-stride", "lhs-input-stride", "output-stride"},
               {{"runtime-element-count", "size_t"}, {"output-buffer", "float *"},
                {"lhs-input-buffer", "const uint8_t *"}, {"rhs-input-buffer", "const uint8_t *"},
                {"rhs-input-stride", "size_t"}, {"source-byte-stride", "size_t"},
                {"destination-byte-stride", "size_t"}, {"lhs-input-stride", "size_t"}, {"output-stride", "size_t"}},
               "q4_0_q8_0_gemm", "cuda-ggml-q4_0-q8_0-gemm-callable-c-abi.v1",
               "tcrv_cuda_gemv_q4_0_q8_0|tcrv_cuda_gemm_q4_0_q8_0", "tcrv_cuda_host_gemm_q4_0_q8_0",
               "decode-gemv-bulk-copy(nc<=8)|prefill-gemm-tcgen05-i8(nc>8)", "hbm|tensor",
               "gemv: 32 lane partials + butterfly; gemm: ascending blocks per element; fused fold"});
  // the integer core of the Q4_0 x Q8_0 block dot as a kernel of its own: offset-binary nibble
  // decode, products against the two activation halves, widening reduction onto a seed
  // (test/Conversion/RVV/rvv-to-emitc-packed-i4-offset-binary-x-i8-product-reduce.mlir)
  t.push_back({"tcrv_rvv.packed_i4_offset_binary_x_i8_product",
               withKind("signed_packed_i4_offset_binary_x_i8_product",
                        {{"product_relation", false, "offset-binary-i4mf4-x-i8mf4x2-to-i16mf2", 0}}),
               "",
               {"tcrv_rvv.load", "tcrv_rvv.load", "tcrv_rvv.load", "tcrv_rvv.packed_i4_offset_binary_x_i8_product",
                "tcrv_rvv.standalone_reduce", "tcrv_rvv.store"},
               {},
               {{"lhs-input-buffer", "const int8_t *"}, {"rhs-input-buffer", "const int8_t *"},
                {"rhs-input-buffer", "const int8_t *"}, {"accumulator-input-buffer", "const int32_t *"},
                {"output-buffer", "int32_t *"}, {"runtime-element-count", "size_t"}},
               "q4_0_q8_0_integer_core", "cuda-q4_0-q8_0-integer-core-callable-c-abi.v1",
               "tcrv_cuda_q4_0_q8_0_integer_core", "tcrv_cuda_host_q4_0_q8_0_integer_core", "single-cta-reduction",
               "latency", ""});
  {
    // one weight row against M activation columns, M a compile-time attribute (1..16)
    RouteEntry e{"tcrv_rvv.q4_0_q8_0_gemm_tile", withKind("ggml_q4_0_q8_0_gemm_tile", kQ4Q8Facts), "",
                 {"tcrv_rvv.q4_0_q8_0_gemm_tile"},
                 {"lhs-input-buffer", "rhs-input-buffer", "rhs-input-stride", "output-buffer", "runtime-element-count"},
                 {{"runtime-element-count", "size_t"}, {"output-buffer", "float *"},
                  {"lhs-input-buffer", "const uint8_t *"}, {"rhs-input-buffer", "const uint8_t *"},
                  {"rhs-input-stride", "size_t"}},
                 "q4_0_q8_0_gemm_tile", "cuda-ggml-q4_0-q8_0-gemm-tile-callable-c-abi.v1",
                 "tcrv_cuda_gemv_q4_0_q8_0|tcrv_cuda_gemm_q4_0_q8_0", "tcrv_cuda_host_gemm_tile_q4_0_q8_0",
                 "block-dot-strict-order(cols<=8)|prefill-gemm-tcgen05-i8(cols>8)", "hbm|tensor",
                 "sumf = fma((float)sumi * d_x, d_y, sumf), ascending blocks, per column"};
    e.constantArgs = {{"activation_cols", 1, 16}};
    t.push_back(e);
  }
  return t;
}

// element type of `!tcrv_rvv.vector<f32, "m1">`
std::string vectorElementType(const std::string &type) {
  const std::string key = "!tcrv_rvv.vector<";
  size_t b = type.find(key);
  if (b == std::string::npos)
    return {};
  size_t e = type.find_first_of(",>", b + key.size());
  return type.substr(b + key.size(), e - b - key.size());
}

std::string factMismatch(const Op &op, const RouteEntry &e) {
  for (const Fact &f : e.facts) {
    if (f.isInteger) {
      long long v = 0;
      if (!op.intAttr(f.key, v))
        return "missing integer attribute '" + f.key + "'";
      if (v != f.integer)
        return "'" + f.key + "' must be " + std::to_string(f.integer) + ", got " + std::to_string(v);
    } else {
      const Attr *a = op.attr(f.key);
      if (!a || a->kind != Attr::String)
        return "missing string attribute '" + f.key + "'";
      if (a->str != f.str)
        return "'" + f.key + "' must be \"" + f.str + "\", got \"" + a->str + "\"";
    }
  }
  for (const RouteEntry::ConstantArg &c : e.constantArgs) {
    long long v = 0;
    if (!op.intAttr(c.attr, v))
      return "missing integer attribute '" + c.attr + "'";
    if (v < c.lo || v > c.hi)
      return "'" + c.attr + "' must lie in " + std::to_string(c.lo) + ".." + std::to_string(c.hi) + ", got " +
             std::to_string(v);
  }
  return {};
}

}  // namespace

const std::vector<RouteEntry> &routeTable() {
  static const std::vector<RouteEntry> table = buildTable();
  return table;
}

// Finds the table entry for a compute op; `why` explains a miss.
const RouteEntry *selectRoute(const Op &computeOp, std::string &why) {
  std::string lastMismatch;
  bool sawOp = false;
  std::string elem;
  if (!computeOp.resultTypes.empty())
    elem = vectorElementType(computeOp.resultTypes[0]);
  for (const RouteEntry &e : routeTable()) {
    if (e.opName != computeOp.name)
      continue;
    sawOp = true;
    std::string m = factMismatch(computeOp, e);
    if (!m.empty()) {
      lastMismatch = m;
      continue;
    }
    if (!e.elementType.empty() && e.elementType != elem) {
      lastMismatch = "no kernel for element type '" + elem + "'";
      continue;
    }
    return &e;
  }
  why = sawOp ? "op " + computeOp.name + ": " + lastMismatch
              : "the CUDA provider has no kernel for op '" + computeOp.name + "'";
  return nullptr;
}

}  // namespace cuda
}  // namespace tcrv
