// Header / descriptor / stub / manifest export for the CUDA provider's emission plans.
#include "tcrv/CUDATarget.h"

#include <sstream>

#include "tcrv/CUDAPlugin.h"

namespace tcrv {
namespace cuda {

namespace {

std::string comparePlans(const VariantEmissionPlan &carried, const VariantEmissionPlan &fresh) {
  auto diff = [](const std::string &what, const std::string &a, const std::string &b) -> std::string {
    return a == b ? std::string() : "stale emission plan: " + what + " is \"" + a + "\", the typed body gives \"" + b + "\"";
  };
  std::string d;
  if (!(d = diff("origin", carried.originPlugin, fresh.originPlugin)).empty()) return d;
  if (!(d = diff("kernel", carried.kernelSymbol, fresh.kernelSymbol)).empty()) return d;
  if (!(d = diff("emission_kind", carried.emissionKind, fresh.emissionKind)).empty()) return d;
  if (!(d = diff("route_id", carried.routeID, fresh.routeID)).empty()) return d;
  if (!(d = diff("runtime_abi_kind", carried.runtimeABIKind, fresh.runtimeABIKind)).empty()) return d;
  if (!(d = diff("runtime_abi_name", carried.runtimeABIName, fresh.runtimeABIName)).empty()) return d;
  if (!(d = diff("runtime_glue_role", carried.runtimeGlueRole, fresh.runtimeGlueRole)).empty()) return d;
  if (!(d = diff("artifact_kind", carried.artifactKind, fresh.artifactKind)).empty()) return d;
  if (!(d = diff("lowering_boundary", carried.loweringBoundary, fresh.loweringBoundary)).empty()) return d;
  if (!(d = diff("entry_symbol", carried.entrySymbol, fresh.entrySymbol)).empty()) return d;
  if (!(d = diff("launcher_symbol", carried.launcherSymbol, fresh.launcherSymbol)).empty()) return d;
  if (!(d = diff("role", toString(carried.role), toString(fresh.role))).empty()) return d;
  if (carried.abiParameters.size() != fresh.abiParameters.size())
    return "stale emission plan: abi_parameters count differs from the typed body";
  for (size_t i = 0; i < fresh.abiParameters.size(); ++i) {
    const auto &a = carried.abiParameters[i], &b = fresh.abiParameters[i];
    if (a.cName != b.cName || a.cType != b.cType || a.role != b.role || a.ownership != b.ownership)
      return "stale emission plan: abi parameter #" + std::to_string(i) + " (" + a.cName + ") does not match the typed body";
  }
  if (carried.metadata.size() != fresh.metadata.size())
    return "stale emission plan: metadata entry count differs from the typed body";
  for (size_t i = 0; i < fresh.metadata.size(); ++i)
    if (carried.metadata[i] != fresh.metadata[i])
      return "stale emission plan: metadata '" + carried.metadata[i].first + "' is \"" + carried.metadata[i].second +
             "\", the typed body gives '" + fresh.metadata[i].first + "' = \"" + fresh.metadata[i].second + "\"";
  return {};
}

}  // namespace

Error collectCoherentPlans(const Op &module, const ExtensionPluginRegistry &registry, std::vector<PlannedVariant> &out) {
  for (const Op *kernel : module.children("tcrv.exec.kernel")) {
    for (const Op *diag : kernel->children("tcrv.exec.diagnostic")) {
      if (diag->strAttr("reason") != "emission_plan")
        continue;
      VariantEmissionPlan carried;
      if (Error e = diagnosticOpToPlan(*diag, carried))
        return e;
      if (!carried.supported)
        return Error("variant @" + carried.variantSymbol + " has an unsupported emission plan: " + carried.diagnostic);
      const Op *variant = nullptr;
      for (const Op *v : kernel->children("tcrv.exec.variant"))
        if (v->symbol == carried.variantSymbol)
          variant = v;
      if (!variant)
        return Error("emission plan targets @" + carried.variantSymbol + ", which is not a variant of kernel @" +
                     kernel->symbol);
      const ExtensionPlugin *plugin = registry.lookup(carried.originPlugin);
      if (!plugin)
        return Error("no provider named \"" + carried.originPlugin + "\" is registered");
      VariantEmissionPlan fresh;
      if (Error e = plugin->buildVariantEmissionPlan({kernel, variant}, fresh))
        return e;
      if (!fresh.supported)
        return Error("the typed body no longer supports the carried plan: " + fresh.diagnostic);
      const std::string d = comparePlans(carried, fresh);
      if (!d.empty())
        return Error(d);
      out.push_back({kernel, variant, carried});
    }
  }
  if (out.empty())
    return Error("the module carries no emission plan (run --tcrv-materialize-emission-plans first)");
  return Error::success();
}

std::string cPrototype(const VariantEmissionPlan &plan) {
  std::ostringstream os;
  std::string ret = "void";
  for (const auto &kv : plan.metadata)
    if (kv.first == "tcrv_cuda.return_type")
      ret = kv.second;
  os << ret << " " << plan.entrySymbol << "(";
  for (size_t i = 0; i < plan.abiParameters.size(); ++i) {
    const auto &p = plan.abiParameters[i];
    const bool pointer = !p.cType.empty() && p.cType.back() == '*';
    os << (i ? ", " : "") << p.cType << (pointer ? "" : " ") << p.cName;
  }
  os << ")";
  return os.str();
}

std::string exportHeaderArtifact(const VariantEmissionPlan &plan) {
  std::ostringstream os;
  os << "// tianchenrv.cuda.selected_variant: @" << plan.variantSymbol << "\n";
  os << "// tianchenrv.cuda.source_kernel: " << plan.kernelSymbol << "\n";
  os << "// tianchenrv.cuda.origin: " << plan.originPlugin << "\n";
  os << "// tianchenrv.cuda.selected_path_role: " << toString(plan.role) << "\n";
  os << "// tianchenrv.cuda.runtime_abi_kind: " << plan.runtimeABIKind << "\n";
  os << "// tianchenrv.cuda.runtime_abi_name: " << plan.runtimeABIName << "\n";
  os << "// tianchenrv.cuda.route_mapping: " << plan.routeID << "\n";
  os << "// tianchenrv.cuda.emission_kind: " << plan.emissionKind << "\n";
  os << "// tianchenrv.cuda.artifact_kind: " << plan.artifactKind << "\n";
  os << "// tianchenrv.cuda.lowering_boundary: " << plan.loweringBoundary << "\n";
  for (const auto &kv : plan.metadata) {
    std::string key = kv.first;
    const std::string prefix = "tcrv_cuda.";
    if (key.compare(0, prefix.size(), prefix) == 0)
      key = key.substr(prefix.size());
    os << "// tianchenrv.cuda." << key << ": " << kv.second << "\n";
  }
  os << "#include <stddef.h>\n#include <stdint.h>\n";
  os << "#ifdef __cplusplus\nextern \"C\" {\n#endif\n";
  os << cPrototype(plan) << ";\n";
  os << "#ifdef __cplusplus\n}\n#endif\n";
  return os.str();
}

static std::string jsonEscape(const std::string &s) {
  std::string out;
  for (char c : s) {
    if (c == '"' || c == '\\')
      out.push_back('\\');
    out.push_back(c);
  }
  return out;
}

std::string exportLaunchDescriptor(const VariantEmissionPlan &plan) {
  std::ostringstream os;
  os << "{\"artifact_kind\": \"" << plan.artifactKind << "\", \"entry_symbol\": \"" << plan.entrySymbol
     << "\", \"launcher_symbol\": \"" << plan.launcherSymbol << "\", \"library\": \"libtcrv_cuda.so\""
     << ", \"runtime_abi_name\": \"" << plan.runtimeABIName << "\", \"route_id\": \"" << plan.routeID
     << "\", \"kernel\": \"" << plan.kernelSymbol << "\", \"variant\": \"" << plan.variantSymbol << "\", \"parameters\": [";
  for (size_t i = 0; i < plan.abiParameters.size(); ++i) {
    const auto &p = plan.abiParameters[i];
    os << (i ? ", " : "") << "{\"c_name\": \"" << p.cName << "\", \"c_type\": \"" << p.cType << "\", \"role\": \""
       << p.role << "\"}";
  }
  os << "], \"metadata\": {";
  for (size_t i = 0; i < plan.metadata.size(); ++i)
    os << (i ? ", " : "") << "\"" << jsonEscape(plan.metadata[i].first) << "\": \"" << jsonEscape(plan.metadata[i].second)
       << "\"";
  os << "}}\n";
  return os.str();
}

// A translation unit that defines the reference-named entry point on top of the
// host-pointer C ABI; what `tcrv-opt --tcrv-rvv-lower-to-emitc | mlir-translate --mlir-to-cpp`
// yields in the reference (generated RVV C), here a call into the prebuilt library.
std::string exportLaunchStubCpp(const VariantEmissionPlan &plan) {
  std::string host, constants;
  for (const auto &kv : plan.metadata) {
    if (kv.first == "tcrv_cuda.host_pointer_symbol")
      host = kv.second;
    if (kv.first == "tcrv_cuda.constant_arguments")
      constants = kv.second;
  }
  std::ostringstream os;
  os << "#include <stddef.h>\n#include <stdint.h>\n#include <stdio.h>\n#include <stdlib.h>\n";
  os << "#include \"tcrv_emitc_host.h\"\n";
  os << "// tcrv_cuda.route=" << plan.routeID << " runtime_abi=" << plan.runtimeABIName << "\n";
  if (host == plan.entrySymbol) {
    os << "// the prebuilt library already defines " << plan.entrySymbol << "\n";
    return os.str();
  }
  os << "extern \"C\" " << cPrototype(plan) << " {\n";
  const bool returnsStatus = host.compare(0, 15, "tcrv_cuda_host_") == 0;
  os << "  " << (returnsStatus ? "const int status = " : "") << host << "(";
  for (size_t i = 0; i < plan.abiParameters.size(); ++i)
    os << (i ? ", " : "") << plan.abiParameters[i].cName;
  // compile-time parameters of the reference kernel ("name=value;..."): trailing literals
  for (size_t b = 0; b < constants.size();) {
    size_t e = constants.find(';', b);
    if (e == std::string::npos)
      e = constants.size();
    const std::string item = constants.substr(b, e - b);
    const size_t eq = item.find('=');
    os << ", /*" << item.substr(0, eq) << "=*/" << item.substr(eq == std::string::npos ? item.size() : eq + 1);
    b = e + 1;
  }
  os << ");\n";
  if (returnsStatus) {
    os << "  if (status != 0) {\n    fprintf(stderr, \"" << plan.entrySymbol
       << ": %s\\n\", tcrv_cuda_status_string(status));\n    abort();\n  }\n";
  }
  os << "}\n";
  return os.str();
}

std::string exportManifestLine(const VariantEmissionPlan &plan) {
  std::ostringstream os;
  os << "kernel=@" << plan.kernelSymbol << " variant=@" << plan.variantSymbol << " origin=" << plan.originPlugin
     << " role=\"" << toString(plan.role) << "\" status=" << (plan.supported ? "supported" : "unsupported")
     << " route=" << plan.routeID << " emission_kind=" << plan.emissionKind << " artifact_kind=" << plan.artifactKind
     << " runtime_abi_name=" << plan.runtimeABIName << " entry=" << plan.entrySymbol
     << " launcher=" << plan.launcherSymbol << "\n";
  return os.str();
}

// ------------------------------------------------------------------ provider hooks

const char *const kBundleIndexFileName = "tianchenrv-target-artifact-bundle.index";

Error configureCUDATargetSupportExtensionBundle(ExtensionBundle &bundle) {
  bundle.addRequiredDialectName("tcrv.exec");
  bundle.addRequiredDialectName("tcrv_rvv");
  bundle.addLoweringBoundaryOp(kBoundaryOp);
  if (Error e = bundle.addTargetArtifactExporter({kRouteId, kArtifactKind, "object", ".json", exportLaunchDescriptor}))
    return e;
  return bundle.addTargetArtifactExporter({kRouteId, "c-header", "header", ".h", exportHeaderArtifact});
}

Error registerCUDATargetSupportTranslateRoutes(TargetTranslateRouteRegistry &registry) {
  TargetTranslateRoute route;
  route.routeID = "tcrv-cuda-launch-to-cpp";
  route.description = "C++ translation unit that defines the reference-named entry point over the prebuilt library";
  route.targetArtifactRouteID = kRouteId;
  route.exportFn = [](const Op &module, const ExtensionPluginRegistry &plugins, std::ostream &os) -> Error {
    std::vector<PlannedVariant> planned;
    if (Error e = collectCoherentPlans(module, plugins, planned))
      return e;
    for (const auto &pv : planned) {
      if (pv.plan.routeID != kRouteId)
        return Error("translate route 'tcrv-cuda-launch-to-cpp' serves route '" + std::string(kRouteId) +
                     "', the plan of @" + pv.plan.variantSymbol + " names '" + pv.plan.routeID + "'");
      os << exportLaunchStubCpp(pv.plan);
    }
    return Error::success();
  };
  return registry.registerRoute(std::move(route));
}

Error collectBundleArtifacts(const Op &module, const ExtensionPluginRegistry &plugins,
                             const ExtensionBundleRegistry &bundles, std::vector<BundleArtifact> &out) {
  std::vector<PlannedVariant> planned;
  if (Error e = collectCoherentPlans(module, plugins, planned))
    return e;
  for (const auto &pv : planned) {
    const ExtensionBundle *bundle = bundles.lookupPluginBundle(pv.plan.originPlugin);
    if (!bundle)
      return Error("provider '" + pv.plan.originPlugin + "' registered no target-support bundle");
    bool any = false;
    for (const char *role : {"object", "artifact", "header"}) {
      const TargetArtifactExporter *ex = bundle->lookupExporter(pv.plan.routeID, role);
      if (!ex)
        continue;
      if (std::string(role) != "header" && ex->artifactKind != pv.plan.artifactKind)
        return Error("route id '" + pv.plan.routeID + "' does not support artifact_kind '" + pv.plan.artifactKind +
                     "'; registered artifact_kind is '" + ex->artifactKind + "'");
      BundleArtifact a;
      a.componentRole = role;
      a.exporter = ex;
      a.plan = pv.plan;
      a.contents = ex->exportFn(pv.plan);
      a.fileName = "artifact-" + std::to_string(out.size()) + "-" + ex->artifactKind + "-" + ex->routeID + ex->fileExtension;
      out.push_back(std::move(a));
      any = true;
    }
    if (!any)
      return Error("bundle '" + bundle->getBundleID() + "' has no exporter for route '" + pv.plan.routeID + "'");
  }
  return Error::success();
}

static std::string quoted(const std::string &s) { return "\"" + jsonEscape(s) + "\""; }

std::string renderBundleIndex(const std::vector<BundleArtifact> &artifacts) {
  std::ostringstream os;
  os << "tianchenrv.target_artifact_bundle.version: 1\n";
  os << "bundle_status: \"complete\"\n";
  os << "artifact_count: " << artifacts.size() << "\n";
  for (size_t i = 0; i < artifacts.size(); ++i) {
    const BundleArtifact &a = artifacts[i];
    const VariantEmissionPlan &p = a.plan;
    os << "artifact[" << i << "]:\n";
    os << "  file_name: " << quoted(a.fileName) << "\n";
    os << "  component_group: " << quoted(p.kernelSymbol + "." + p.variantSymbol) << "\n";
    os << "  component_role: " << quoted(a.componentRole) << "\n";
    os << "  external_abi_name: " << quoted(p.runtimeABIName) << "\n";
    os << "  selected_variant: @" << p.variantSymbol << "\n";
    os << "  role: " << quoted(toString(p.role)) << "\n";
    os << "  artifact_kind: " << quoted(a.exporter->artifactKind) << "\n";
    os << "  route: " << quoted(p.routeID) << "\n";
    os << "  owner: " << quoted(p.originPlugin) << "\n";
    os << "  runtime_abi: " << quoted(p.entrySymbol) << "\n";
    os << "  runtime_abi_kind: " << quoted(p.runtimeABIKind) << "\n";
    os << "  runtime_abi_name: " << quoted(p.runtimeABIName) << "\n";
    os << "  runtime_abi_parameter_count: " << p.abiParameters.size() << "\n";
    for (size_t j = 0; j < p.abiParameters.size(); ++j) {
      const RuntimeABIParameter &q = p.abiParameters[j];
      os << "  runtime_abi_parameter[" << j << "]:\n";
      os << "    c_name: " << quoted(q.cName) << "\n";
      os << "    c_type: " << quoted(q.cType) << "\n";
      os << "    role: " << quoted(q.role) << "\n";
      os << "    ownership: " << quoted(q.ownership) << "\n";
    }
    for (size_t j = 0; j < p.metadata.size(); ++j) {
      os << "  artifact_metadata[" << j << "]:\n";
      os << "    key: " << quoted(p.metadata[j].first) << "\n";
      os << "    value: " << quoted(p.metadata[j].second) << "\n";
    }
    os << "  handoff_kind: " << quoted(p.emissionKind) << "\n";
    os << "  evidence_role: " << quoted(a.componentRole == "header" ? "c-abi-declaration" : "launch-descriptor") << "\n";
  }
  return os.str();
}

}  // namespace cuda
}  // namespace tcrv
