// tcrv-translate look-alike: exports target artifacts from a module that carries emission
// plans.  Flag names follow the reference driver (tools/tcrv-translate/tcrv-translate.cpp:40-48,
// 448-482):
//   --tcrv-export-emission-manifest
//   --tcrv-export-target-header-artifact
//   --tcrv-export-target-artifact          (the launch descriptor, JSON)
//   --tcrv-export-target-artifact-bundle   with --tcrv-target-artifact-bundle-output-dir=<dir>:
//                                          every artifact of every plan as a file, plus an index
//   --<translate route id>                 routes the providers registered (tcrv-cuda-launch-to-cpp:
//                                          C++ stub defining the reference-named entry point)
//   --tcrv-disable-builtin-plugins         empty provider registry (every export then fails closed)
// The driver owns no target knowledge: exporters and translate routes reach it through the
// providers' configureTargetSupportExtensionBundle / registerTargetSupportTranslateRoutes
// hooks.  Every export first re-derives the plan from the typed body and refuses a stale one.
#include <sys/stat.h>

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

static bool isDirectory(const std::string &path) {
  struct stat st;
  return stat(path.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}

static Error writeFile(const std::string &path, const std::string &contents) {
  std::ofstream f(path, std::ios::binary | std::ios::trunc);
  if (!f)
    return Error("cannot create '" + path + "'");
  f << contents;
  f.close();
  if (!f)
    return Error("cannot write '" + path + "'");
  return Error::success();
}

int main(int argc, char **argv) {
  std::string mode, input = "-", bundleDir;
  bool builtin = true;
  const std::string dirFlag = "--tcrv-target-artifact-bundle-output-dir";
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    if (a == "--tcrv-disable-builtin-plugins")
      builtin = false;
    else if (a.compare(0, dirFlag.size() + 1, dirFlag + "=") == 0)
      bundleDir = a.substr(dirFlag.size() + 1);
    else if (a == dirFlag && i + 1 < argc)
      bundleDir = argv[++i];
    else if (a.rfind("--", 0) == 0) {
      if (!mode.empty())
        return fail("more than one translation requested ('" + mode + "' and '" + a + "')");
      mode = a;
    } else
      input = a;
  }
  if (mode.empty())
    return fail("no translation requested");

  ExtensionPluginRegistry plugins;
  if (builtin)
    registerBuiltinPlugins(plugins);
  ExtensionBundleRegistry bundles;
  if (Error e = registerExtensionBundles(plugins, bundles))
    return fail(e.message);
  TargetTranslateRouteRegistry routes;
  if (Error e = registerTargetTranslateRoutes(plugins, routes))
    return fail(e.message);

  const bool fixed = mode == "--tcrv-export-emission-manifest" || mode == "--tcrv-export-target-header-artifact" ||
                     mode == "--tcrv-export-target-artifact" || mode == "--tcrv-export-target-artifact-bundle";
  const TargetTranslateRoute *route = fixed ? nullptr : routes.lookup(mode.substr(2));
  if (!fixed && !route)
    return fail("unknown option '" + mode + "'");

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

  if (route) {
    std::ostringstream out;
    if (Error e = route->exportFn(*parsed.module, plugins, out))
      return fail(e.message);
    std::cout << out.str();
    return 0;
  }
  if (mode == "--tcrv-export-emission-manifest") {
    std::vector<cuda::PlannedVariant> planned;
    if (Error e = cuda::collectCoherentPlans(*parsed.module, plugins, planned))
      return fail(e.message);
    for (const auto &pv : planned)
      std::cout << cuda::exportManifestLine(pv.plan);
    return 0;
  }
  // the three artifact exports go through the exporters of the owning provider's bundle
  std::vector<cuda::BundleArtifact> artifacts;
  if (Error e = cuda::collectBundleArtifacts(*parsed.module, plugins, bundles, artifacts))
    return fail(e.message);
  if (mode == "--tcrv-export-target-artifact-bundle") {
    if (bundleDir.empty())
      return fail("TianChen-RV target artifact bundle export failed: --tcrv-target-artifact-bundle-output-dir is required");
    if (!isDirectory(bundleDir))
      return fail("TianChen-RV target artifact bundle export failed: output directory '" + bundleDir +
                  "' does not exist");
    for (const auto &a : artifacts)
      if (Error e = writeFile(bundleDir + "/" + a.fileName, a.contents))
        return fail("TianChen-RV target artifact bundle export failed: " + e.message);
    if (Error e = writeFile(bundleDir + "/" + cuda::kBundleIndexFileName, cuda::renderBundleIndex(artifacts)))
      return fail("TianChen-RV target artifact bundle export failed: " + e.message);
    std::cout << "tianchenrv.target_artifact_bundle_export: complete\n";
    std::cout << "index_file: \"" << cuda::kBundleIndexFileName << "\"\n";
    return 0;
  }
  const std::string want = mode == "--tcrv-export-target-header-artifact" ? "header" : "object";
  for (const auto &a : artifacts)
    if (a.componentRole == want)
      std::cout << a.contents;
  return 0;
}
