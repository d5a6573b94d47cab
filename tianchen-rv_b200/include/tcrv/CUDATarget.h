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

}  // namespace cuda
}  // namespace tcrv
