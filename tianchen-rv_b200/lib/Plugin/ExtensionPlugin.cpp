// Provider registry, the envelope checks every provider shares, and the plan carrier op.
#include "tcrv/ExtensionPlugin.h"

#include <cctype>
#include <map>
#include <set>

namespace tcrv {

const char *toString(VariantEmissionRole role) {
  switch (role) {
    case VariantEmissionRole::DispatchCase:
      return "dispatch case";
    case VariantEmissionRole::Fallback:
      return "dispatch fallback";
    case VariantEmissionRole::DirectCall:
      return "direct call";
  }
  return "direct call";
}

Error ExtensionPluginRegistry::registerPlugin(std::shared_ptr<const ExtensionPlugin> plugin) {
  if (!plugin || plugin->getName().empty())
    return Error("cannot register a provider without a name");
  if (lookup(plugin->getName()))
    return Error("provider '" + plugin->getName() + "' is already registered");
  plugins.push_back(std::move(plugin));
  return Error::success();
}

const ExtensionPlugin *ExtensionPluginRegistry::lookup(const std::string &origin) const {
  for (const auto &p : plugins)
    if (p->getName() == origin && p->isEnabled())
      return p.get();
  return nullptr;
}

std::vector<std::string> ExtensionPluginRegistry::names() const {
  std::vector<std::string> out;
  for (const auto &p : plugins)
    out.push_back(p->getName());
  return out;
}

// ------------------------------------------------------------------ target support

Error ExtensionPlugin::configureTargetSupportExtensionBundle(ExtensionBundle &) const { return Error::success(); }
Error ExtensionPlugin::registerTargetSupportTranslateRoutes(TargetTranslateRouteRegistry &) const {
  return Error::success();
}

Error ExtensionBundle::addTargetArtifactExporter(TargetArtifactExporter exporter) {
  if (exporter.routeID.empty() || exporter.artifactKind.empty() || exporter.componentRole.empty() || !exporter.exportFn)
    return Error("bundle '" + bundleID + "': an artifact exporter needs a route id, an artifact kind, a component role "
                 "and an export function");
  if (lookupExporter(exporter.routeID, exporter.componentRole))
    return Error("bundle '" + bundleID + "': route '" + exporter.routeID + "' already has a '" + exporter.componentRole +
                 "' exporter");
  exporters.push_back(std::move(exporter));
  return Error::success();
}

const TargetArtifactExporter *ExtensionBundle::lookupExporter(const std::string &routeID,
                                                              const std::string &componentRole) const {
  for (const auto &e : exporters)
    if (e.routeID == routeID && e.componentRole == componentRole)
      return &e;
  return nullptr;
}

Error ExtensionBundleRegistry::registerBundle(ExtensionBundle bundle) {
  if (bundle.getBundleID().empty() || bundle.getPluginName().empty())
    return Error("an extension bundle needs an id and a provider name");
  for (const auto &b : bundles)
    if (b.getBundleID() == bundle.getBundleID() || b.getPluginName() == bundle.getPluginName())
      return Error("extension bundle '" + bundle.getBundleID() + "' (provider '" + bundle.getPluginName() +
                   "') is already registered");
  bundles.push_back(std::move(bundle));
  return Error::success();
}

const ExtensionBundle *ExtensionBundleRegistry::lookupPluginBundle(const std::string &pluginName) const {
  for (const auto &b : bundles)
    if (b.getPluginName() == pluginName)
      return &b;
  return nullptr;
}

Error TargetTranslateRouteRegistry::registerRoute(TargetTranslateRoute route) {
  if (route.routeID.empty() || !route.exportFn)
    return Error("a translate route needs an id and an export function");
  if (lookup(route.routeID))
    return Error("translate route '" + route.routeID + "' is already registered");
  routes.push_back(std::move(route));
  return Error::success();
}

const TargetTranslateRoute *TargetTranslateRouteRegistry::lookup(const std::string &routeID) const {
  for (const auto &r : routes)
    if (r.routeID == routeID)
      return &r;
  return nullptr;
}

Error registerExtensionBundles(const ExtensionPluginRegistry &plugins, ExtensionBundleRegistry &bundles) {
  for (const auto &p : plugins.getPlugins()) {
    if (!p->isEnabled())
      continue;
    ExtensionBundle bundle(p->getName() + "-bundle", p->getName());
    if (Error e = p->configureTargetSupportExtensionBundle(bundle))
      return e;
    if (Error e = bundles.registerBundle(std::move(bundle)))
      return e;
  }
  return Error::success();
}

Error registerTargetTranslateRoutes(const ExtensionPluginRegistry &plugins, TargetTranslateRouteRegistry &routes) {
  for (const auto &p : plugins.getPlugins())
    if (p->isEnabled())
      if (Error e = p->registerTargetSupportTranslateRoutes(routes))
        return e;
  return Error::success();
}

// ------------------------------------------------------------------ envelope checks

static std::string where(const VariantRequest &r) {
  return "kernel @" + (r.kernel ? r.kernel->symbol : std::string("?")) + " variant @" +
         (r.variant ? r.variant->symbol : std::string("?")) + ": ";
}

Error verifyVariantEnvelope(const VariantRequest &r) {
  if (!r.kernel || !r.variant)
    return Error("missing kernel or variant");
  if (r.kernel->symbol.empty())
    return Error("tcrv.exec.kernel needs a symbol name");
  if (r.variant->symbol.empty())
    return Error(where(r) + "tcrv.exec.variant needs a symbol name");
  if (r.variant->strAttr("origin").empty())
    return Error(where(r) + "variant needs a non-empty 'origin'");
  const Attr *req = r.variant->attr("requires");
  if (!req || req->kind != Attr::Array || req->elements.empty())
    return Error(where(r) + "variant needs a non-empty 'requires' array");
  for (const Attr &e : req->elements) {
    if (e.kind != Attr::SymbolRef)
      return Error(where(r) + "'requires' must hold symbol references");
    bool found = false;
    for (const Op *cap : r.kernel->children("tcrv.exec.capability"))
      found = found || cap->symbol == e.str;
    if (!found)
      return Error(where(r) + "required capability @" + e.str + " is not declared in the kernel");
  }
  return Error::success();
}

Error checkCapabilityRequires(const VariantRequest &r) {
  if (Error e = verifyVariantEnvelope(r))
    return e;
  for (const Attr &e : r.variant->attr("requires")->elements) {
    for (const Op *cap : r.kernel->children("tcrv.exec.capability")) {
      if (cap->symbol != e.str)
        continue;
      if (cap->strAttr("id").empty() || cap->strAttr("kind").empty())
        return Error(where(r) + "capability @" + cap->symbol + " needs 'id' and 'kind'");
      if (cap->strAttr("status") != "available")
        return Error(where(r) + "required capability @" + cap->symbol + " is not available (status \"" +
                     cap->strAttr("status") + "\")");
    }
  }
  return Error::success();
}

static bool safeCIdentifier(const std::string &s) {
  if (s.empty() || !(std::isalpha(static_cast<unsigned char>(s[0])) || s[0] == '_'))
    return false;
  for (char c : s)
    if (!(std::isalnum(static_cast<unsigned char>(c)) || c == '_'))
      return false;
  static const std::set<std::string> keywords = {"int",  "float", "double", "char",   "void",  "const", "if",
                                                 "else", "for",   "while",  "return", "short", "long",  "struct"};
  return keywords.count(s) == 0;
}

// C types a role may carry.
static bool cTypeAllowed(const std::string &role, const std::string &cType) {
  static const std::set<std::string> inputBuffers = {"const int8_t *",  "const uint8_t *", "const int16_t *",
                                                     "const int32_t *", "const int64_t *", "const float *",
                                                     "const double *"};
  static const std::set<std::string> outputBuffers = {"int8_t *",  "uint8_t *", "int16_t *", "int32_t *",
                                                      "int64_t *", "float *",   "double *"};
  if (role == "lhs-input-buffer" || role == "rhs-input-buffer" || role == "accumulator-input-buffer")
    return inputBuffers.count(cType) != 0;
  if (role == "output-buffer")
    return outputBuffers.count(cType) != 0;
  if (role == "runtime-element-count" || role == "output-stride" || role == "lhs-input-stride" ||
      role == "rhs-input-stride" || role == "source-byte-stride" || role == "destination-byte-stride")
    return cType == "size_t";
  if (role == "dequant-scale-value")
    return cType == "float";
  if (role == "rhs-scalar-value")
    return cType == "int32_t" || cType == "int64_t" || cType == "float";
  return false;  // unknown role
}

Error collectRuntimeABI(const Op &variant, std::vector<RuntimeABIParameter> &out) {
  std::set<std::string> names;
  for (const Op *v : variant.children("tcrv_rvv.runtime_abi_value")) {
    RuntimeABIParameter p;
    p.ssaName = v->results.empty() ? std::string() : v->results[0];
    p.cName = v->strAttr("c_name");
    p.cType = v->strAttr("c_type");
    p.role = v->strAttr("role");
    p.ownership = v->strAttr("ownership");
    const std::string at = "runtime_abi_value " + p.ssaName + " (line " + std::to_string(v->line) + "): ";
    if (p.ssaName.empty())
      return Error(at + "needs a result");
    if (!safeCIdentifier(p.cName))
      return Error(at + "c_name \"" + p.cName + "\" is not a safe C identifier");
    if (!names.insert(p.cName).second)
      return Error(at + "c_name \"" + p.cName + "\" is used twice");
    if (p.ownership != "target-export-abi-owned")
      return Error(at + "ownership must be \"target-export-abi-owned\"");
    if (p.role.empty())
      return Error(at + "needs a role");
    if (!cTypeAllowed(p.role, p.cType))
      return Error(at + "c_type \"" + p.cType + "\" is not allowed for role \"" + p.role + "\"");
    out.push_back(p);
  }
  if (out.empty())
    return Error("variant @" + variant.symbol + " declares no runtime ABI values");
  return Error::success();
}

std::string entrySymbolFor(const std::string &kernelSymbol, const std::string &variantSymbol) {
  return "tcrv_emitc_" + kernelSymbol + "_" + variantSymbol;
}

VariantEmissionRole emissionRoleOf(const VariantRequest &r) {
  if (const Op *dispatch = r.kernel->firstChild("tcrv.exec.dispatch")) {
    for (const auto &c : dispatch->body) {
      if (c->symbol != r.variant->symbol)
        continue;
      if (c->name == "tcrv.exec.case")
        return VariantEmissionRole::DispatchCase;
      if (c->name == "tcrv.exec.fallback")
        return VariantEmissionRole::Fallback;
    }
  }
  return VariantEmissionRole::DirectCall;
}

// ------------------------------------------------------------------ plan carrier op

static Attr strAttrOf(const std::string &v) {
  Attr a;
  a.kind = Attr::String;
  a.str = v;
  a.text = "\"" + v + "\"";
  return a;
}

static Attr arrayOf(const std::vector<std::string> &items) {
  Attr a;
  a.kind = Attr::Array;
  a.text = "[";
  for (size_t i = 0; i < items.size(); ++i) {
    Attr e = strAttrOf(items[i]);
    a.text += (i ? ", " : "") + e.text;
    a.elements.push_back(e);
  }
  a.text += "]";
  return a;
}

std::unique_ptr<Op> planToDiagnosticOp(const VariantEmissionPlan &plan) {
  auto op = std::make_unique<Op>();
  op->name = "tcrv.exec.diagnostic";
  auto add = [&](const std::string &k, const Attr &a) { op->attrs.emplace_back(k, a); };
  std::vector<std::string> abi, meta;
  for (const auto &p : plan.abiParameters)
    abi.push_back(p.cName + "|" + p.cType + "|" + p.role + "|" + p.ownership);
  for (const auto &kv : plan.metadata)
    meta.push_back(kv.first + "=" + kv.second);
  add("abi_parameters", arrayOf(abi));
  add("artifact_kind", strAttrOf(plan.artifactKind));
  add("emission_kind", strAttrOf(plan.emissionKind));
  add("entry_symbol", strAttrOf(plan.entrySymbol));
  add("kernel", strAttrOf(plan.kernelSymbol));
  add("launcher_symbol", strAttrOf(plan.launcherSymbol));
  add("lowering_boundary", strAttrOf(plan.loweringBoundary));
  add("metadata", arrayOf(meta));
  add("origin", strAttrOf(plan.originPlugin));
  add("reason", strAttrOf("emission_plan"));
  add("role", strAttrOf(toString(plan.role)));
  add("route_id", strAttrOf(plan.routeID));
  add("runtime_abi_kind", strAttrOf(plan.runtimeABIKind));
  add("runtime_abi_name", strAttrOf(plan.runtimeABIName));
  add("runtime_glue_role", strAttrOf(plan.runtimeGlueRole));
  add("status", strAttrOf(plan.supported ? "supported" : "unsupported"));
  if (!plan.supported)
    add("diagnostic", strAttrOf(plan.diagnostic));
  Attr target;
  target.kind = Attr::SymbolRef;
  target.str = plan.variantSymbol;
  target.text = "@" + plan.variantSymbol;
  add("target", target);
  return op;
}

Error diagnosticOpToPlan(const Op &d, VariantEmissionPlan &out) {
  if (d.name != "tcrv.exec.diagnostic" || d.strAttr("reason") != "emission_plan")
    return Error("not an emission-plan diagnostic");
  out = VariantEmissionPlan();
  out.supported = d.strAttr("status") == "supported";
  out.diagnostic = d.strAttr("diagnostic");
  out.artifactKind = d.strAttr("artifact_kind");
  out.emissionKind = d.strAttr("emission_kind");
  out.entrySymbol = d.strAttr("entry_symbol");
  out.kernelSymbol = d.strAttr("kernel");
  out.launcherSymbol = d.strAttr("launcher_symbol");
  out.loweringBoundary = d.strAttr("lowering_boundary");
  out.originPlugin = d.strAttr("origin");
  out.routeID = d.strAttr("route_id");
  out.runtimeABIKind = d.strAttr("runtime_abi_kind");
  out.runtimeABIName = d.strAttr("runtime_abi_name");
  out.runtimeGlueRole = d.strAttr("runtime_glue_role");
  const std::string role = d.strAttr("role");
  out.role = role == "dispatch case"       ? VariantEmissionRole::DispatchCase
             : role == "dispatch fallback" ? VariantEmissionRole::Fallback
                                           : VariantEmissionRole::DirectCall;
  const Attr *target = d.attr("target");
  if (!target || target->kind != Attr::SymbolRef)
    return Error("emission plan has no target variant");
  out.variantSymbol = target->str;
  const Attr *abi = d.attr("abi_parameters");
  if (!abi || abi->kind != Attr::Array)
    return Error("emission plan has no abi_parameters");
  for (const Attr &e : abi->elements) {
    std::vector<std::string> parts;
    size_t start = 0;
    while (true) {
      size_t bar = e.str.find('|', start);
      parts.push_back(e.str.substr(start, bar == std::string::npos ? std::string::npos : bar - start));
      if (bar == std::string::npos)
        break;
      start = bar + 1;
    }
    if (parts.size() != 4)
      return Error("malformed abi parameter \"" + e.str + "\"");
    RuntimeABIParameter p;
    p.cName = parts[0], p.cType = parts[1], p.role = parts[2], p.ownership = parts[3];
    out.abiParameters.push_back(p);
  }
  if (const Attr *meta = d.attr("metadata")) {
    for (const Attr &e : meta->elements) {
      size_t eq = e.str.find('=');
      if (eq == std::string::npos)
        return Error("malformed metadata entry \"" + e.str + "\"");
      out.metadata.emplace_back(e.str.substr(0, eq), e.str.substr(eq + 1));
    }
  }
  return Error::success();
}

}  // namespace tcrv
