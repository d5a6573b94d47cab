// The CUDA provider's public pieces: its constants, the route table entry type and the
// factory.  One table entry = one hand-written sm_100a kernel family behind a C-ABI launcher,
// keyed by typed facts (op mnemonic, pinned attribute values, element type, ABI signature).
#pragma once

#include <string>
#include <utility>
#include <vector>

#include "tcrv/ExtensionPlugin.h"

namespace tcrv {
namespace cuda {

extern const char *const kPluginName;       // "cuda-plugin"
extern const char *const kCapabilityId;     // "cuda.sm_100a"
extern const char *const kCapabilityKind;   // "accelerator"
extern const char *const kProtocolAttr;     // boundary attribute naming the construction protocol
extern const char *const kProtocolValue;
extern const char *const kRouteId;
extern const char *const kEmissionKind;
extern const char *const kArtifactKind;
extern const char *const kBoundaryOp;
extern const char *const kRuntimeABIKind;
extern const char *const kGlueRole;

struct Fact {
  std::string key;
  bool isInteger;
  std::string str;
  long long integer;
};

struct RouteEntry {
  std::string opName;                    // typed compute op, e.g. "tcrv_rvv.q4_0_q8_0_gemm"
  std::vector<Fact> facts;               // attribute values the op must carry
  std::string elementType;               // vector element type to match ("" = not applicable)
  std::vector<std::string> bodyOps;      // ops inside the boundary, in order
  std::vector<std::string> operandRoles; // ABI role of each compute-op operand ("" = not checked)
  std::vector<std::pair<std::string, std::string>> abi;  // (role, c_type) in declaration order
  std::string operation;                 // short operation name for the plan
  std::string runtimeABIName;
  std::string launcherSymbol;            // device-pointer C-ABI entry point(s)
  std::string hostSymbol;                // host-pointer twin
  std::string kernelFamily;
  std::string rooflineBound;             // "hbm", "tensor" or both
  std::string foldOrder;                 // fp32 fold convention ("" for non-dot kernels)
  std::string returnType = "void";       // C return type of the entry (soft_max returns its f64 sum)
  // Integer attributes of the compute op that are compile-time parameters of the reference's
  // kernel (e.g. the column count of a GEMM tile): each must lie in [lo, hi] and is passed to
  // the host-pointer entry as a trailing literal argument.
  struct ConstantArg {
    std::string attr;
    long long lo, hi;
  };
  std::vector<ConstantArg> constantArgs = {};
  // What a planner should know about the route beyond its bound, e.g. that a layout is served
  // for compatibility and another one is the fast one ("" = nothing to say).
  std::string layoutNote = "";
};

const std::vector<RouteEntry> &routeTable();
const RouteEntry *selectRoute(const Op &computeOp, std::string &why);

std::shared_ptr<const ExtensionPlugin> createCUDAExtensionPlugin();

}  // namespace cuda
}  // namespace tcrv

// ---- abstract contraction request -> concrete op (the provider picks HOW) ----
namespace tcrv {
namespace cuda {

enum class QuantType { Q4_0, Q8_0 };
enum class MRegime { Decode, Prefill };
enum class ContractionAlgorithm {
  StreamingGemv,   // plain-format weight streaming, dp4a, HBM-bound (decode)
  TensorCoreGemm,  // tcgen05 kind::i8 over the prepared planar layout (prefill)
};

struct ContractionSelection {
  ContractionAlgorithm algorithm;
  const char *algorithmName;         // stamped as tcrv_cuda.contraction_algorithm
  const char *reason;                // stamped as tcrv_cuda.path_selection_reason
  const char *weightLayoutContract;  // stamped as tcrv_cuda.weight_layout_contract
};

// Pure function of the request's facts, the counterpart of the reference's
// selectContractionAlgorithm (include/TianChenRV/Plugin/RVV/RVVContractionPathSelection.h:31-70).
ContractionSelection selectContractionAlgorithm(QuantType quant, MRegime regime);

// Lowers every `tcrv_rvv.quant_contraction` under a CUDA-provider boundary of `kernel` to
// the concrete block-dot op it stands for and stamps the audit attributes
// (lib/Plugin/RVV/RVVLowerQuantContraction.cpp:80-99, :301).  `lowered` counts rewrites.
Error lowerQuantContractions(Op &kernel, int &lowered);

}  // namespace cuda
}  // namespace tcrv
