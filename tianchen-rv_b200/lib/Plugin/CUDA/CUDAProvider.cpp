// The CUDA provider's ExtensionPlugin implementation: legality, readiness, boundary
// validation and realization, and the emission plan.  The route table lives in
// CUDAExtensionPlugin.cpp.
#include <algorithm>
#include <map>
#include <sstream>

#include "tcrv/CUDAPlugin.h"
#include "tcrv/CUDATarget.h"

namespace tcrv {
namespace cuda {
namespace {

std::string where(const VariantRequest &r) {
  return "kernel @" + r.kernel->symbol + " variant @" + r.variant->symbol + ": ";
}

const Op *boundaryOf(const Op &variant) { return variant.firstChild(kBoundaryOp); }

const Op *computeOpOf(const Op &boundary) {
  for (const auto &c : boundary.body)
    if (c->name != "tcrv_rvv.load" && c->name != "tcrv_rvv.store")
      return c.get();
  return nullptr;
}

std::string joinSymbols(const Attr *a) {
  std::string out;
  if (a && a->kind == Attr::Array)
    for (const Attr &e : a->elements)
      out += (out.empty() ? "" : ",") + e.str;
  return out;
}

// element type named by a runtime-ABI buffer type, e.g. "const float *" -> "f32"
std::string elementOfCType(const std::string &cType) {
  if (cType.find("float") != std::string::npos)
    return "f32";
  if (cType.find("int32_t") != std::string::npos)
    return "i32";
  return {};
}

Attr strAttr(const std::string &v) {
  Attr a;
  a.kind = Attr::String;
  a.str = v;
  a.text = "\"" + v + "\"";
  return a;
}

Attr intAttr(long long v, const char *type) {
  Attr a;
  a.kind = Attr::Integer;
  a.integer = v;
  a.text = std::to_string(v) + " : " + type;
  return a;
}

Attr symbolAttr(const std::string &name) {
  Attr a;
  a.kind = Attr::SymbolRef;
  a.str = name;
  a.text = "@" + name;
  return a;
}

class CUDAExtensionPlugin final : public ExtensionPlugin {
public:
  std::string getName() const override { return kPluginName; }
  std::string getVersion() const override { return "sm_100a.v1"; }
  std::vector<PluginCapability> getCapabilities() const override { return {{kCapabilityId, kCapabilityKind}}; }

  bool supportsOperation(const Op &computeOp) const override {
    std::string why;
    return selectRoute(computeOp, why) != nullptr;
  }

  // Envelope + capability identity + runtime ABI: everything that does not need the boundary.
  Error verifyVariantLegality(const VariantRequest &r) const override {
    if (Error e = verifyVariantEnvelope(r))
      return e;
    if (r.variant->strAttr("origin") != kPluginName)
      return Error(where(r) + "origin \"" + r.variant->strAttr("origin") + "\" is not this provider");
    bool hasCuda = false;
    for (const Attr &req : r.variant->attr("requires")->elements)
      for (const Op *cap : r.kernel->children("tcrv.exec.capability"))
        if (cap->symbol == req.str && cap->strAttr("id") == kCapabilityId && cap->strAttr("kind") == kCapabilityKind)
          hasCuda = true;
    if (!hasCuda)
      return Error(where(r) + "variant must require a capability {id = \"" + kCapabilityId + "\", kind = \"" +
                   kCapabilityKind + "\"}");
    std::vector<RuntimeABIParameter> abi;
    return collectRuntimeABI(*r.variant, abi);
  }

  Error estimateVariantCost(const VariantRequest &r, VariantCostEstimate &out) const override {
    const RouteEntry *route = nullptr;
    if (Error e = resolve(r, route))
      return e;
    // Relative cost per byte or per op moved; HBM-bound kernels are priced by bytes.
    out.relativeCost = route->rooflineBound == "hbm" ? 1.0 : 0.5;
    out.explanation = "sm_100a " + route->kernelFamily + " (" + route->rooflineBound + "-bound)";
    return Error::success();
  }

  Error checkVariantEmissionReadiness(const VariantRequest &r, VariantEmissionStatus &out) const override {
    out.ready = false;
    if (Error e = checkCapabilityRequires(r)) {
      out.reason = e.message;
      return Error::success();
    }
    if (Error e = validateSelectedLoweringBoundary(r)) {
      out.reason = e.message;
      return Error::success();
    }
    out.ready = true;
    out.reason = "selected lowering boundary validated";
    return Error::success();
  }

  Error validateSelectedLoweringBoundary(const VariantRequest &r) const override {
    const RouteEntry *route = nullptr;
    return resolve(r, route);
  }

  Error buildVariantEmissionPlan(const VariantRequest &r, VariantEmissionPlan &plan) const override {
    plan = VariantEmissionPlan();
    plan.originPlugin = kPluginName;
    plan.kernelSymbol = r.kernel ? r.kernel->symbol : std::string();
    plan.variantSymbol = r.variant ? r.variant->symbol : std::string();
    const RouteEntry *route = nullptr;
    Error err = checkCapabilityRequires(r);
    if (!err)
      err = resolve(r, route);
    if (err) {
      plan.supported = false;
      plan.diagnostic = err.message;
      plan.role = (r.kernel && r.variant) ? emissionRoleOf(r) : VariantEmissionRole::DirectCall;
      return Error::success();
    }
    plan.supported = true;
    plan.role = emissionRoleOf(r);
    plan.emissionKind = kEmissionKind;
    plan.routeID = kRouteId;
    plan.runtimeABIKind = kRuntimeABIKind;
    plan.runtimeABIName = route->runtimeABIName;
    plan.runtimeGlueRole = kGlueRole;
    plan.artifactKind = kArtifactKind;
    plan.loweringBoundary = kBoundaryOp;
    plan.entrySymbol = entrySymbolFor(plan.kernelSymbol, plan.variantSymbol);
    plan.launcherSymbol = route->launcherSymbol;
    (void)collectRuntimeABI(*r.variant, plan.abiParameters);

    const Op *compute = computeOpOf(*boundaryOf(*r.variant));
    auto meta = [&](const std::string &k, const std::string &v) { plan.metadata.emplace_back(k, v); };
    meta("cuda_selected_body_operation", route->operation);
    meta("cuda_selected_body_typed_compute_op", route->opName);
    if (!route->elementType.empty())
      meta("tcrv_cuda.element_type", route->elementType);
    std::string facts;
    for (const Fact &f : route->facts)
      facts += (facts.empty() ? "" : ";") + f.key + "=" + (f.isInteger ? std::to_string(f.integer) : f.str);
    meta("tcrv_cuda.typed_facts", facts);
    std::string binding;
    for (const auto &p : plan.abiParameters)
      binding += (binding.empty() ? "" : ";") + p.cName + "=" + p.role + ":" + p.cType;
    meta("tcrv_cuda.route_operand_binding_operands", binding);
    meta("tcrv_cuda.launcher_symbol", route->launcherSymbol);
    meta("tcrv_cuda.host_pointer_symbol", route->hostSymbol);
    meta("tcrv_cuda.kernel_family", route->kernelFamily);
    meta("tcrv_cuda.roofline_bound", route->rooflineBound);
    if (!route->foldOrder.empty())
      meta("tcrv_cuda.fp32_fold_order", route->foldOrder);
    if (!route->layoutNote.empty())
      meta("tcrv_cuda.layout_note", route->layoutNote);
    if (route->returnType != "void")
      meta("tcrv_cuda.return_type", route->returnType);
    if (!route->constantArgs.empty()) {
      std::string consts;
      for (const RouteEntry::ConstantArg &c : route->constantArgs) {
        long long v = 0;
        (void)compute->intAttr(c.attr, v);  // presence and range were checked when the route was selected
        consts += (consts.empty() ? "" : ";") + c.attr + "=" + std::to_string(v);
      }
      meta("tcrv_cuda.constant_arguments", consts);
    }
    meta("tcrv_cuda.target_arch", "sm_100a");
    meta("tcrv_cuda.required_capabilities", joinSymbols(r.variant->attr("requires")));
    meta("tcrv_cuda.required_header_declarations", "stddef.h,stdint.h");
    meta("tcrv_cuda.pointer_space", "entry:host;launcher:device");
    (void)compute;
    return Error::success();
  }

  // Realizes `tcrv_rvv.typed_binary_pre_realized_body` (the reference's pre-realized
  // elementwise body, test/Target/RVV/pre-realized-selected-body-artifact-add.mlir:25) into
  // setvl + boundary + load/load/binary/store.  A variant that already has a boundary is
  // left alone.
  Error configureTargetSupportExtensionBundle(ExtensionBundle &bundle) const override {
    return configureCUDATargetSupportExtensionBundle(bundle);
  }
  Error registerTargetSupportTranslateRoutes(TargetTranslateRouteRegistry &registry) const override {
    return registerCUDATargetSupportTranslateRoutes(registry);
  }

  Error materializeSelectedLoweringBoundary(Op &kernel, Op &variant) const override {
    VariantRequest r{&kernel, &variant};
    if (Error e = verifyVariantLegality(r))
      return e;
    if (boundaryOf(variant))
      return validateSelectedLoweringBoundary(r);
    size_t index = variant.body.size();
    for (size_t i = 0; i < variant.body.size(); ++i)
      if (variant.body[i]->name == "tcrv_rvv.typed_binary_pre_realized_body")
        index = i;
    if (index == variant.body.size())
      return Error(where(r) + "no selected lowering boundary and no pre-realized body to realize");
    const Op pre = std::move(*variant.body[index]);
    if (pre.operands.size() != 4)
      return Error(where(r) + "typed_binary_pre_realized_body takes lhs, rhs, out, n");
    if (pre.strAttr("op_kind") != "add")
      return Error(where(r) + "the CUDA provider realizes op_kind \"add\" only, got \"" + pre.strAttr("op_kind") + "\"");
    long long sew = 0;
    if (!pre.intAttr("sew", sew) || sew != 32)
      return Error(where(r) + "pre-realized body needs sew = 32");
    std::vector<RuntimeABIParameter> abi;
    if (Error e = collectRuntimeABI(variant, abi))
      return e;
    std::string elem;
    for (const auto &p : abi)
      if (p.ssaName == pre.operands[0])
        elem = elementOfCType(p.cType);
    if (elem.empty())
      return Error(where(r) + "cannot derive the element type of the pre-realized body from its lhs buffer");
    const std::string vec = "!tcrv_rvv.vector<" + elem + ", \"m1\">";
    const std::string abiTy = "!tcrv_rvv.runtime_abi_value", vlTy = "!tcrv_rvv.vl";

    auto setvl = std::make_unique<Op>();
    setvl->results = {"%vl"};
    setvl->name = "tcrv_rvv.setvl";
    setvl->operands = {pre.operands[3]};
    setvl->attrs.emplace_back("lmul", strAttr("m1"));
    if (const Attr *pol = pre.attr("policy"))
      setvl->attrs.emplace_back("policy", *pol);
    setvl->attrs.emplace_back("sew", intAttr(32, "i64"));
    setvl->operandTypes = {"index"};
    setvl->resultTypes = {vlTy};

    auto boundary = std::make_unique<Op>();
    boundary->name = kBoundaryOp;
    boundary->operands = {"%vl"};
    boundary->hasRegion = true;
    boundary->attrs.emplace_back(kProtocolAttr, strAttr(kProtocolValue));
    boundary->attrs.emplace_back("lmul", strAttr("m1"));
    boundary->attrs.emplace_back("origin", strAttr(kPluginName));
    if (const Attr *pol = pre.attr("policy"))
      boundary->attrs.emplace_back("policy", *pol);
    boundary->attrs.emplace_back("required_capabilities", *variant.attr("requires"));
    boundary->attrs.emplace_back("selected_path_role", strAttr(toString(emissionRoleOf(r))));
    boundary->attrs.emplace_back("selected_variant", symbolAttr(variant.symbol));
    boundary->attrs.emplace_back("sew", intAttr(32, "i64"));
    boundary->attrs.emplace_back("source_kernel", strAttr(kernel.symbol));
    boundary->attrs.emplace_back("status", strAttr("selected-lowering-boundary"));
    boundary->operandTypes = {vlTy};

    auto mk = [&](const std::string &name, std::vector<std::string> results, std::vector<std::string> operands,
                  std::vector<std::string> operandTypes, std::vector<std::string> resultTypes) {
      auto op = std::make_unique<Op>();
      op->name = name;
      op->results = std::move(results);
      op->operands = std::move(operands);
      op->operandTypes = std::move(operandTypes);
      op->resultTypes = std::move(resultTypes);
      return op;
    };
    boundary->body.push_back(mk("tcrv_rvv.load", {"%a"}, {pre.operands[0], "%vl"}, {abiTy, vlTy}, {vec}));
    boundary->body.push_back(mk("tcrv_rvv.load", {"%b"}, {pre.operands[1], "%vl"}, {abiTy, vlTy}, {vec}));
    auto bin = mk("tcrv_rvv.binary", {"%sum"}, {"%a", "%b", "%vl"}, {vec, vec, vlTy}, {vec});
    bin->attrs.emplace_back("kind", strAttr("add"));
    boundary->body.push_back(std::move(bin));
    boundary->body.push_back(mk("tcrv_rvv.store", {}, {pre.operands[2], "%sum", "%vl"}, {abiTy, vec, vlTy}, {}));

    variant.body[index] = std::move(setvl);
    variant.body.insert(variant.body.begin() + index + 1, std::move(boundary));
    return validateSelectedLoweringBoundary(r);
  }

private:
  // Full fail-closed validation; on success `route` is the selected table entry.
  Error resolve(const VariantRequest &r, const RouteEntry *&route) const {
    if (Error e = verifyVariantLegality(r))
      return e;
    const auto boundaries = r.variant->children(kBoundaryOp);
    if (boundaries.size() != 1)
      return Error(where(r) + "expected exactly one " + kBoundaryOp + " boundary, found " +
                   std::to_string(boundaries.size()));
    const Op &b = *boundaries[0];
    auto need = [&](const std::string &key, const std::string &want) -> Error {
      if (b.strAttr(key) != want)
        return Error(where(r) + "boundary attribute '" + key + "' must be \"" + want + "\", got \"" + b.strAttr(key) +
                     "\"");
      return Error::success();
    };
    if (Error e = need("source_kernel", r.kernel->symbol))
      return e;
    if (Error e = need("origin", kPluginName))
      return e;
    if (Error e = need("status", "selected-lowering-boundary"))
      return e;
    if (Error e = need(kProtocolAttr, kProtocolValue))
      return e;
    if (Error e = need("selected_path_role", toString(emissionRoleOf(r))))
      return e;
    const Attr *sel = b.attr("selected_variant");
    if (!sel || sel->kind != Attr::SymbolRef || sel->str != r.variant->symbol)
      return Error(where(r) + "boundary attribute 'selected_variant' must be @" + r.variant->symbol);
    if (joinSymbols(b.attr("required_capabilities")) != joinSymbols(r.variant->attr("requires")))
      return Error(where(r) + "boundary 'required_capabilities' must equal the variant's 'requires'");
    const Op *setvl = r.variant->firstChild("tcrv_rvv.setvl");
    if (!setvl || setvl->results.empty() || b.operands.empty() || b.operands[0] != setvl->results[0])
      return Error(where(r) + "the boundary must consume the !tcrv_rvv.vl token of the variant's setvl");

    const Op *compute = computeOpOf(b);
    if (!compute)
      return Error(where(r) + "the boundary holds no compute op");
    std::string why;
    route = selectRoute(*compute, why);
    if (!route)
      return Error(where(r) + why);
    // body shape
    if (b.body.size() != route->bodyOps.size())
      return Error(where(r) + "boundary body must be [" + joinOps(route->bodyOps) + "]");
    for (size_t i = 0; i < b.body.size(); ++i)
      if (b.body[i]->name != route->bodyOps[i])
        return Error(where(r) + "boundary body must be [" + joinOps(route->bodyOps) + "], op #" + std::to_string(i) +
                     " is " + b.body[i]->name);
    // runtime ABI signature, in declaration order
    std::vector<RuntimeABIParameter> abi;
    if (Error e = collectRuntimeABI(*r.variant, abi))
      return e;
    if (abi.size() != route->abi.size())
      return Error(where(r) + "runtime ABI must declare " + std::to_string(route->abi.size()) + " values for " +
                   route->operation + ", found " + std::to_string(abi.size()));
    std::map<std::string, std::string> roleOf;
    for (size_t i = 0; i < abi.size(); ++i) {
      if (abi[i].role != route->abi[i].first || abi[i].cType != route->abi[i].second)
        return Error(where(r) + "runtime ABI value #" + std::to_string(i) + " (" + abi[i].cName + ") must be {" +
                     route->abi[i].first + ", " + route->abi[i].second + "}, got {" + abi[i].role + ", " +
                     abi[i].cType + "}");
      roleOf[abi[i].ssaName] = abi[i].role;
    }
    // operand wiring of block ops: each operand must be the ABI value with the expected role
    for (size_t i = 0; i < route->operandRoles.size(); ++i) {
      if (i >= compute->operands.size())
        return Error(where(r) + route->opName + " is missing operand #" + std::to_string(i));
      if (roleOf[compute->operands[i]] != route->operandRoles[i])
        return Error(where(r) + route->opName + " operand #" + std::to_string(i) + " must be the " +
                     route->operandRoles[i] + " value");
    }
    // elementwise bodies: loads read the input buffers, the store writes the output buffer
    if (route->bodyOps.size() > 1) {
      for (const auto &c : b.body) {
        if (c->name == "tcrv_rvv.load" &&
            (c->operands.empty() || roleOf[c->operands[0]].find("input-buffer") == std::string::npos))
          return Error(where(r) + "tcrv_rvv.load must read an input buffer");
        if (c->name == "tcrv_rvv.store" && (c->operands.empty() || roleOf[c->operands[0]] != "output-buffer"))
          return Error(where(r) + "tcrv_rvv.store must write the output buffer");
      }
    }
    return Error::success();
  }

  static std::string joinOps(const std::vector<std::string> &ops) {
    std::string out;
    for (const auto &o : ops)
      out += (out.empty() ? "" : ", ") + o;
    return out;
  }
};

}  // namespace

std::shared_ptr<const ExtensionPlugin> createCUDAExtensionPlugin() {
  return std::make_shared<CUDAExtensionPlugin>();
}

}  // namespace cuda

void registerBuiltinPlugins(ExtensionPluginRegistry &registry) {
  (void)registry.registerPlugin(cuda::createCUDAExtensionPlugin());
}

}  // namespace tcrv
