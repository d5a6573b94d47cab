// tcrv-translate look-alike: exports target artifacts from a module that carries emission
// plans.  Flag names follow the reference driver (tools/tcrv-translate/tcrv-translate.cpp:448-482):
//   --tcrv-export-emission-manifest
//   --tcrv-export-target-header-artifact
//   --tcrv-export-target-artifact          (the launch descriptor, JSON)
//   --tcrv-cuda-launch-to-cpp              (C++ stub defining the reference-named entry point)
// Every export first re-derives the plan from the typed body and refuses a stale one.
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>

#include "tcrv/CUDATarget.h"

using namespace tcrv;

static int fail(const std::string &msg) {
  std::cerr << "tcrv-translate: error: " << msg << "\n";
  return 1;
}

int main(int argc, char **argv) {
  std::string mode, input = "-";
  bool builtin = true;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    if (a == "--tcrv-export-emission-manifest" || a == "--tcrv-export-target-header-artifact" ||
        a == "--tcrv-export-target-artifact" || a == "--tcrv-cuda-launch-to-cpp")
      mode = a;
    else if (a == "--tcrv-disable-builtin-plugins")
      builtin = false;
    else if (a.rfind("--", 0) == 0)
      return fail("unknown option '" + a + "'");
    else
      input = a;
  }
  if (mode.empty())
    return fail("no translation requested");
  std::ostringstream ss;
  if (input == "-") {
    ss << std::cin.rdbuf();
  } else {
    std::ifstream f(input);
    if (!f)
      return fail("cannot open '" + input + "'");
    ss << f.rdbuf();
  }
  ParseResult parsed = parseFixture(ss.str());
  if (!parsed.module)
    return fail(parsed.error);
  ExtensionPluginRegistry registry;
  if (builtin)
    registerBuiltinPlugins(registry);
  std::vector<cuda::PlannedVariant> planned;
  if (Error e = cuda::collectCoherentPlans(*parsed.module, registry, planned))
    return fail(e.message);
  for (const auto &pv : planned) {
    if (mode == "--tcrv-export-emission-manifest")
      std::cout << cuda::exportManifestLine(pv.plan);
    else if (mode == "--tcrv-export-target-header-artifact")
      std::cout << cuda::exportHeaderArtifact(pv.plan);
    else if (mode == "--tcrv-export-target-artifact")
      std::cout << cuda::exportLaunchDescriptor(pv.plan);
    else
      std::cout << cuda::exportLaunchStubCpp(pv.plan);
  }
  return 0;
}
