// Provider ("extension plugin") interface of the drop-in boundary, in plain C++.
//
// It mirrors the method set of the reference's plugin interface
// (include/TianChenRV/Plugin/ExtensionPlugin.h:653-693) and the fields of its emission plan
// (include/TianChenRV/Plugin/ExtensionPlugin.h:440-572) with fixture ops (tcrv/Fixture.h) in
// place of MLIR operations and an Error value in place of llvm::Error.  Selection goes by
// typed facts only -- op identity, attribute values, element types, runtime-ABI roles and C
// types, capability records -- never by kernel or variant names.
#pragma once

#include <functional>
#include <iosfwd>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "tcrv/Fixture.h"

namespace tcrv {

// Success when `message` is empty; otherwise a one-line, human-readable diagnostic.
struct Error {
  std::string message;
  Error() = default;
  explicit Error(std::string m) : message(std::move(m)) {}
  explicit operator bool() const { return !message.empty(); }  // true == failure, like llvm::Error
  static Error success() { return Error(); }
};

struct PluginCapability {
  std::string id;    // e.g. "cuda.sm_100a"
  std::string kind;  // e.g. "accelerator"
};

// One parameter of the exported C entry point, in declaration order
// (include/TianChenRV/Support/RuntimeABI.h:26-74).
struct RuntimeABIParameter {
  std::string ssaName;  // "%lhs"
  std::string cName, cType, role, ownership;
};

enum class VariantEmissionRole { DispatchCase, Fallback, DirectCall };
const char *toString(VariantEmissionRole role);

struct VariantRequest {
  const Op *kernel = nullptr;   // tcrv.exec.kernel
  const Op *variant = nullptr;  // tcrv.exec.variant inside it
};

struct VariantCostEstimate {
  double relativeCost = 0.0;  // lower is better
  std::string explanation;
};

struct VariantEmissionStatus {
  bool ready = false;
  std::string reason;
};

struct VariantEmissionPlan {
  bool supported = false;
  VariantEmissionRole role = VariantEmissionRole::DirectCall;
  std::string originPlugin, kernelSymbol, variantSymbol;
  std::string emissionKind;        // e.g. "prebuilt-sm100a-kernel-c-abi-launch"
  std::string routeID;             // lowering pipeline / route family id
  std::string runtimeABIKind;      // "plugin-owned-runtime-abi"
  std::string runtimeABIName;      // e.g. "cuda-q4_0-q8_0-gemm-callable-c-abi.v1"
  std::string runtimeGlueRole;
  std::string artifactKind;        // "cuda-sm100a-launch-descriptor"
  std::string loweringBoundary;    // boundary op name, "tcrv_rvv.with_vl"
  std::string entrySymbol;         // tcrv_emitc_<kernel>_<variant>
  std::string launcherSymbol;      // device-pointer C-ABI function behind it
  std::vector<RuntimeABIParameter> abiParameters;
  std::vector<std::pair<std::string, std::string>> metadata;  // ordered key/value facts
  std::string diagnostic;          // set when !supported
};

class ExtensionPluginRegistry;

// ---- target side of a provider -----------------------------------------------------------
//
// One exporter of a provider's target support: turns an emission plan of route `routeID` into
// one artifact of `artifactKind` (the reference's exporter registry by route id,
// lib/Target/RVV/RVVTargetSupportBundle.cpp:1738-1806).
struct TargetArtifactExporter {
  std::string routeID;
  std::string artifactKind;
  std::string componentRole;  // "header", "object" or "artifact": how a bundle index lists the file
  std::string fileExtension;  // including the dot
  std::function<std::string(const VariantEmissionPlan &)> exportFn;
};

// What a provider contributes to the target side, filled by
// ExtensionPlugin::configureTargetSupportExtensionBundle (the reference's ExtensionBundle,
// include/TianChenRV/Plugin/ExtensionBundle.h:26-61).
class ExtensionBundle {
public:
  ExtensionBundle() = default;
  ExtensionBundle(std::string bundleID, std::string pluginName)
      : bundleID(std::move(bundleID)), pluginName(std::move(pluginName)) {}
  const std::string &getBundleID() const { return bundleID; }
  const std::string &getPluginName() const { return pluginName; }
  const std::vector<std::string> &getRequiredDialectNames() const { return requiredDialectNames; }
  const std::vector<std::string> &getLoweringBoundaryOps() const { return loweringBoundaryOps; }
  const std::vector<TargetArtifactExporter> &getTargetArtifactExporters() const { return exporters; }
  void addRequiredDialectName(const std::string &name) { requiredDialectNames.push_back(name); }
  void addLoweringBoundaryOp(const std::string &name) { loweringBoundaryOps.push_back(name); }
  // Fails on a second exporter for the same (route, component role).
  Error addTargetArtifactExporter(TargetArtifactExporter exporter);
  const TargetArtifactExporter *lookupExporter(const std::string &routeID, const std::string &componentRole) const;

private:
  std::string bundleID, pluginName;
  std::vector<std::string> requiredDialectNames, loweringBoundaryOps;
  std::vector<TargetArtifactExporter> exporters;
};

class ExtensionBundleRegistry {
public:
  Error registerBundle(ExtensionBundle bundle);
  const ExtensionBundle *lookupPluginBundle(const std::string &pluginName) const;
  const std::vector<ExtensionBundle> &getBundles() const { return bundles; }

private:
  std::vector<ExtensionBundle> bundles;
};

// A named translation of the tcrv-translate driver that a provider registers
// (include/TianChenRV/Target/TargetTranslateRegistration.h:20-58): `--<routeID>` on the command
// line runs exportFn over the module.
struct TargetTranslateRoute {
  std::string routeID;
  std::string description;
  std::function<Error(const Op &module, const ExtensionPluginRegistry &plugins, std::ostream &os)> exportFn;
  std::string targetArtifactRouteID;  // the plan route this translation serves ("" = any)
};

class TargetTranslateRouteRegistry {
public:
  Error registerRoute(TargetTranslateRoute route);
  const TargetTranslateRoute *lookup(const std::string &routeID) const;
  const std::vector<TargetTranslateRoute> &getRoutes() const { return routes; }
  size_t size() const { return routes.size(); }

private:
  std::vector<TargetTranslateRoute> routes;
};

class ExtensionPlugin {
public:
  virtual ~ExtensionPlugin() = default;

  virtual std::string getName() const = 0;
  virtual std::string getVersion() const { return {}; }
  virtual std::vector<PluginCapability> getCapabilities() const = 0;
  virtual bool isEnabled() const { return true; }
  // Does this provider have a kernel for the typed compute op (identity + facts)?
  virtual bool supportsOperation(const Op &computeOp) const = 0;
  virtual Error verifyVariantLegality(const VariantRequest &request) const = 0;
  virtual Error estimateVariantCost(const VariantRequest &request, VariantCostEstimate &out) const = 0;
  virtual Error checkVariantEmissionReadiness(const VariantRequest &request, VariantEmissionStatus &out) const = 0;
  virtual Error buildVariantEmissionPlan(const VariantRequest &request, VariantEmissionPlan &out) const = 0;
  // Expands a pre-realized typed body into setvl + boundary + load/compute/store in place.
  virtual Error materializeSelectedLoweringBoundary(Op &kernel, Op &variant) const = 0;
  virtual Error validateSelectedLoweringBoundary(const VariantRequest &request) const = 0;
  // Target support (include/TianChenRV/Plugin/ExtensionPlugin.h:689-692): the provider names the
  // dialects and boundary ops its bundle needs and hands over its artifact exporters, and
  // registers the translations the driver exposes for it.  A provider without target support
  // keeps the defaults, which add nothing.
  virtual Error configureTargetSupportExtensionBundle(ExtensionBundle &bundle) const;
  virtual Error registerTargetSupportTranslateRoutes(TargetTranslateRouteRegistry &registry) const;
};

class ExtensionPluginRegistry {
public:
  Error registerPlugin(std::shared_ptr<const ExtensionPlugin> plugin);
  const ExtensionPlugin *lookup(const std::string &origin) const;
  std::vector<std::string> names() const;
  const std::vector<std::shared_ptr<const ExtensionPlugin>> &getPlugins() const { return plugins; }
  bool empty() const { return plugins.empty(); }

private:
  std::vector<std::shared_ptr<const ExtensionPlugin>> plugins;
};

// The built-in provider table: one line per provider, as in the reference's
// lib/Plugin/Builtin/BuiltinExtensionPlugins.cpp:34-42.
void registerBuiltinPlugins(ExtensionPluginRegistry &registry);
// One bundle per registered provider, configured by the provider itself, and the translate
// routes the providers register (lib/Target/BuiltinTargetTranslateRoutes.cpp in the reference).
Error registerExtensionBundles(const ExtensionPluginRegistry &plugins, ExtensionBundleRegistry &bundles);
Error registerTargetTranslateRoutes(const ExtensionPluginRegistry &plugins, TargetTranslateRouteRegistry &routes);

// ---- checks shared by every provider (the envelope is dialect-level in the reference) ----

// Variant has a non-empty origin and a non-empty `requires` array whose symbols resolve to
// tcrv.exec.capability ops of the same kernel (lib/Dialect/Exec/IR/ExecOps.cpp:787-843).
Error verifyVariantEnvelope(const VariantRequest &request);
// Every required capability has status "available" (--tcrv-check-capability-requires).
Error checkCapabilityRequires(const VariantRequest &request);
// Collects and validates the runtime ABI values of a variant in declaration order: role,
// safe unique c_name, c_type allowed for the role, ownership "target-export-abi-owned"
// (lib/Dialect/RVV/IR/RVVDialectControlOps.cpp:38-154, lib/Dialect/RVV/IR/RVVDialect.cpp:2144-2202).
Error collectRuntimeABI(const Op &variant, std::vector<RuntimeABIParameter> &out);
// `tcrv_emitc_<kernel>_<variant>` (lib/Conversion/RVV/RVVToEmitC.cpp:165-172).
std::string entrySymbolFor(const std::string &kernelSymbol, const std::string &variantSymbol);
// Role of a variant from the kernel's dispatch op: case / fallback / direct call.
VariantEmissionRole emissionRoleOf(const VariantRequest &request);

// ---- plan <-> tcrv.exec.diagnostic (the carrier op the passes write and translate reads) ----
std::unique_ptr<Op> planToDiagnosticOp(const VariantEmissionPlan &plan);
Error diagnosticOpToPlan(const Op &diag, VariantEmissionPlan &out);

}  // namespace tcrv
