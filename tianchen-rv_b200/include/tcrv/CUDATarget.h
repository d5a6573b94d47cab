// Target-side exports of the CUDA provider: header artifact, launch descriptor, launch stub
// and emission manifest, all produced from an emission plan that is first re-derived from
// the typed body and compared with the plan the module carries (a stale or edited plan
// fails the export, as in the reference's tamper tests,
// test/Target/RVV/pre-realized-selected-body-artifact-add.mlir:4-10).
#pragma once

#include <string>
#include <vector>

#include "tcrv/ExtensionPlugin.h"

namespace tcrv {
namespace cuda {

struct PlannedVariant {
  const Op *kernel = nullptr;
  const Op *variant = nullptr;
  VariantEmissionPlan plan;  // as carried by the module
};

// Finds every supported emission plan in the module and checks it against a fresh plan.
Error collectCoherentPlans(const Op &module, const ExtensionPluginRegistry &registry,
                           std::vector<PlannedVariant> &out);

std::string cPrototype(const VariantEmissionPlan &plan);
std::string exportHeaderArtifact(const VariantEmissionPlan &plan);
std::string exportLaunchDescriptor(const VariantEmissionPlan &plan);
std::string exportLaunchStubCpp(const VariantEmissionPlan &plan);
std::string exportManifestLine(const VariantEmissionPlan &plan);

// The provider's two target-support hooks end here: the bundle receives the dialect names, the
// boundary op and the header / launch-descriptor exporters of the provider's route; the
// translate registry receives `tcrv-cuda-launch-to-cpp` (the counterpart of the reference's
// `tcrv-rvv-emitc-to-cpp`, lib/Plugin/RVV/Construction/RVVConstructionProtocol.cpp:174-199).
Error configureCUDATargetSupportExtensionBundle(ExtensionBundle &bundle);
Error registerCUDATargetSupportTranslateRoutes(TargetTranslateRouteRegistry &registry);

// One file of an exported bundle and the record the index holds for it.
struct BundleArtifact {
  std::string fileName, componentRole, contents;
  const TargetArtifactExporter *exporter = nullptr;
  VariantEmissionPlan plan;
};
// Every artifact of every coherent plan of the module, in index order: per plan the object-role
// artifact (the launch descriptor) and then the header, as the reference's bundle lists them
// (test/Target/RVV/pre-realized-selected-body-artifact-runtime-scalar-dual-cmp-mask-and-select-bundle.mlir:44-60).
Error collectBundleArtifacts(const Op &module, const ExtensionPluginRegistry &plugins,
                             const ExtensionBundleRegistry &bundles, std::vector<BundleArtifact> &out);
// The text of `tianchenrv-target-artifact-bundle.index` (field names and order of the
// reference's index writer, lib/Target/TargetArtifactExport.cpp:2939-3018).
std::string renderBundleIndex(const std::vector<BundleArtifact> &artifacts);
extern const char *const kBundleIndexFileName;

}  // namespace cuda
}  // namespace tcrv
