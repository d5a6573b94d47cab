// tcrv-opt look-alike: runs the planning "passes" of the drop-in boundary over a textual
// fixture and prints the resulting module.  Flag names follow the reference driver
// (tools/tcrv-opt/tcrv-opt.cpp:41-139, include/TianChenRV/Transforms/Passes.td):
//   --tcrv-check-capability-requires
//   --tcrv-materialize-selected-lowering-boundaries
//   --tcrv-materialize-emission-plans
//   --tcrv-cuda-lower-quant-contraction   (counterpart of --tcrv-rvv-lower-quant-contraction)
//   --tcrv-disable-builtin-plugins
// Passes run in command-line order over every variant whose origin names a registered
// provider; variants of other origins (e.g. a scalar fallback) are left untouched.
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#include "tcrv/CUDAPlugin.h"
#include "tcrv/ExtensionPlugin.h"

using namespace tcrv;

namespace {

int fail(const std::string &msg) {
  std::cerr << "tcrv-opt: error: " << msg << "\n";
  return 1;
}

std::string readAll(std::istream &in) {
  std::ostringstream ss;
  ss << in.rdbuf();
  return ss.str();
}

}  // namespace

int main(int argc, char **argv) {
  std::vector<std::string> passes;
  std::string input = "-";
  bool builtin = true;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    if (a == "--tcrv-disable-builtin-plugins")
      builtin = false;
    else if (a == "--tcrv-check-capability-requires" || a == "--tcrv-materialize-selected-lowering-boundaries" ||
             a == "--tcrv-materialize-emission-plans" || a == "--tcrv-cuda-lower-quant-contraction")
      passes.push_back(a);
    else if (a == "--help" || a == "-h") {
      std::cout << "usage: tcrv-opt [file|-] [--tcrv-check-capability-requires] "
                   "[--tcrv-materialize-selected-lowering-boundaries] [--tcrv-materialize-emission-plans] "
                   "[--tcrv-cuda-lower-quant-contraction] [--tcrv-disable-builtin-plugins]\n";
      return 0;
    } else if (a.rfind("--", 0) == 0)
      return fail("unknown option '" + a + "'");
    else
      input = a;
  }
  std::string text;
  if (input == "-") {
    text = readAll(std::cin);
  } else {
    std::ifstream f(input);
    if (!f)
      return fail("cannot open '" + input + "'");
    text = readAll(f);
  }
  ParseResult parsed = parseFixture(text);
  if (!parsed.module)
    return fail(parsed.error);
  ExtensionPluginRegistry registry;
  if (builtin)
    registerBuiltinPlugins(registry);

  for (const std::string &pass : passes) {
    for (auto &kop : parsed.module->body) {
      if (kop->name != "tcrv.exec.kernel")
        continue;
      Op &kernel = *kop;
      if (pass == "--tcrv-cuda-lower-quant-contraction") {
        int lowered = 0;
        if (Error e = cuda::lowerQuantContractions(kernel, lowered))
          return fail(e.message);
        continue;
      }
      std::vector<std::unique_ptr<Op>> plans;
      for (auto &vop : kernel.body) {
        if (vop->name != "tcrv.exec.variant")
          continue;
        Op &variant = *vop;
        VariantRequest req{&kernel, &variant};
        if (Error e = verifyVariantEnvelope(req))
          return fail(e.message);
        const ExtensionPlugin *plugin = registry.lookup(variant.strAttr("origin"));
        if (!plugin) {
          // a variant that carries a typed body needs its provider; an empty envelope does not
          if (variant.firstChild("tcrv_rvv.runtime_abi_value") && !builtin)
            return fail("kernel @" + kernel.symbol + " variant @" + variant.symbol + ": no provider named \"" +
                        variant.strAttr("origin") + "\" is registered");
          continue;
        }
        if (pass == "--tcrv-check-capability-requires") {
          if (Error e = checkCapabilityRequires(req))
            return fail(e.message);
        } else if (pass == "--tcrv-materialize-selected-lowering-boundaries") {
          if (Error e = plugin->materializeSelectedLoweringBoundary(kernel, variant))
            return fail(e.message);
        } else {
          VariantEmissionStatus status;
          if (Error e = plugin->checkVariantEmissionReadiness(req, status))
            return fail(e.message);
          if (!status.ready)
            return fail(status.reason);
          VariantEmissionPlan plan;
          if (Error e = plugin->buildVariantEmissionPlan(req, plan))
            return fail(e.message);
          if (!plan.supported)
            return fail(plan.diagnostic);
          plans.push_back(planToDiagnosticOp(plan));
        }
      }
      if (pass == "--tcrv-materialize-emission-plans") {
        // replace earlier plans of the same kernel
        std::vector<std::unique_ptr<Op>> kept;
        for (auto &c : kernel.body)
          if (!(c->name == "tcrv.exec.diagnostic" && c->strAttr("reason") == "emission_plan"))
            kept.push_back(std::move(c));
        kernel.body = std::move(kept);
        for (auto &p : plans)
          kernel.body.push_back(std::move(p));
      }
    }
  }
  std::cout << printOp(*parsed.module);
  return 0;
}
