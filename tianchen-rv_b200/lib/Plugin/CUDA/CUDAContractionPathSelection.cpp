// The provider's answer to an algorithm-uncommitted contraction request
// (`tcrv_rvv.quant_contraction`, include/TianChenRV/Dialect/RVV/IR/RVVOps.td:3975-4046): a
// pure selection function over (quant, m_regime) and the pass body that lowers the request
// to a concrete op with audit attributes, mirroring
// lib/Plugin/RVV/RVVContractionPathSelection.cpp:69-91 and
// lib/Plugin/RVV/RVVLowerQuantContraction.cpp:80-99.
#include "tcrv/CUDAPlugin.h"

namespace tcrv {
namespace cuda {

ContractionSelection selectContractionAlgorithm(QuantType quant, MRegime regime) {
  // Fact 1: is there a tensor-core kernel for this weight format?  (Q4_0 only.)
  // Fact 2: does the regime amortise the operand preparation?  A prefill GEMM reuses every
  //         prepared weight tile across hundreds of columns and is compute-bound; a decode
  //         step reads each weight byte once, so anything but streaming the plain format
  //         adds HBM traffic.
  const bool hasTensorCoreKernel = quant == QuantType::Q4_0;
  if (regime == MRegime::Prefill && hasTensorCoreKernel)
    return {ContractionAlgorithm::TensorCoreGemm, "prefill-gemm-tcgen05-i8", "tensor-core-kept-q4_0-prefill",
            "planar-int8-fp32-scales"};
  if (regime == MRegime::Prefill)
    return {ContractionAlgorithm::StreamingGemv, "decode-gemv-bulk-copy",
            "streaming-decline-q8_0-no-tensor-core-kernel", "plain"};
  return {ContractionAlgorithm::StreamingGemv, "decode-gemv-bulk-copy",
          quant == QuantType::Q4_0 ? "streaming-kept-q4_0-decode-hbm-bound" : "streaming-kept-q8_0-decode-hbm-bound",
          "plain"};
}

namespace {

Attr strAttr(const std::string &v) {
  Attr a;
  a.kind = Attr::String;
  a.str = v;
  a.text = "\"" + v + "\"";
  return a;
}

Error lowerOne(Op &op, const std::string &at) {
  auto needInt = [&](const char *key, long long want) -> Error {
    long long v = 0;
    if (!op.intAttr(key, v) || v != want)
      return Error(at + "quant_contraction needs " + key + " = " + std::to_string(want));
    return Error::success();
  };
  const std::string quant = op.strAttr("quant"), regime = op.strAttr("m_regime");
  if (quant != "q4_0" && quant != "q8_0")
    return Error(at + "quant_contraction: unsupported quant \"" + quant + "\"");
  if (regime != "decode" && regime != "prefill")
    return Error(at + "quant_contraction: m_regime must be \"decode\" or \"prefill\", got \"" + regime + "\"");
  if (op.strAttr("weight_layout") != "plain")
    return Error(at + "quant_contraction takes plain weights (weight_layout = \"plain\")");
  if (op.strAttr("scale_model") != "dual-fp16-per-block-d_x.d_y")
    return Error(at + "quant_contraction: unsupported scale_model \"" + op.strAttr("scale_model") + "\"");
  const bool q4 = quant == "q4_0";
  if (Error e = needInt("qk", 32))
    return e;
  if (Error e = needInt("weight_block_stride", q4 ? 18 : 34))
    return e;
  if (Error e = needInt("activation_block_stride", 34))
    return e;
  if (Error e = needInt("quant_byte_offset", 2))
    return e;
  if (q4)
    if (Error e = needInt("activation_high_byte_offset", 16))
      return e;
  if (op.operands.size() != 6 || op.operandTypes.size() != 6)
    return Error(at + "quant_contraction takes weight, activation, output, n, nc and the vl token");

  const ContractionSelection sel = selectContractionAlgorithm(q4 ? QuantType::Q4_0 : QuantType::Q8_0,
                                                              regime == "prefill" ? MRegime::Prefill : MRegime::Decode);
  // The concrete block dot writes one fp32 and leaves the row/column loops to its caller,
  // so the column-count operand is dropped (as the reference's identity lowering does).
  op.name = q4 ? "tcrv_rvv.q4_0_q8_0_block_dot" : "tcrv_rvv.q8_0_q8_0_block_dot";
  op.operands.erase(op.operands.begin() + 4);
  op.operandTypes.erase(op.operandTypes.begin() + 4);
  std::vector<std::pair<std::string, Attr>> attrs;
  attrs.emplace_back("kind", strAttr(q4 ? "ggml_q4_0_q8_0_block_dot" : "ggml_q8_0_q8_0_block_dot"));
  for (auto &kv : op.attrs) {
    if (kv.first == "quant" || kv.first == "m_regime" || kv.first == "weight_layout" || kv.first == "min_vlen")
      continue;
    attrs.push_back(kv);
  }
  attrs.emplace_back("tcrv_cuda.contraction_algorithm", strAttr(sel.algorithmName));
  attrs.emplace_back("tcrv_cuda.path_selection_reason", strAttr(sel.reason));
  attrs.emplace_back("tcrv_cuda.weight_layout_contract", strAttr(sel.weightLayoutContract));
  op.attrs = std::move(attrs);
  return Error::success();
}

}  // namespace

Error lowerQuantContractions(Op &kernel, int &lowered) {
  for (auto &v : kernel.body) {
    if (v->name != "tcrv.exec.variant" || v->strAttr("origin") != kPluginName)
      continue;
    for (auto &b : v->body) {
      if (b->name != kBoundaryOp)
        continue;
      for (auto &c : b->body) {
        if (c->name != "tcrv_rvv.quant_contraction")
          continue;
        const std::string at = "kernel @" + kernel.symbol + " variant @" + v->symbol + ": ";
        if (Error e = lowerOne(*c, at))
          return e;
        ++lowered;
      }
    }
  }
  return Error::success();
}

}  // namespace cuda
}  // namespace tcrv
