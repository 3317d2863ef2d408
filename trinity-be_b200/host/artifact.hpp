// Compiled-plan artifacts: directory layout source.cu, exports.map, program.so, manifest.json,
// diagnostics.json (src/compile/cuda/mod.rs:62-109 in the reference).
#pragma once

#include <stdexcept>
#include <string>

#include "emit.hpp"

namespace trinity::host {

struct CompileConfig {
  std::string host_compiler;  // default: $CXX or g++
  std::string library_dir;    // default: the configured kernel-library directory
};

// kind: Config | MissingCompiler | MissingLibrary | Io | CompilerFailed | MissingArtifact
struct CompileFailure : std::runtime_error {
  std::string kind, diagnostics_json;
  CompileFailure(const std::string& k, const std::string& what, const std::string& diagnostics)
      : std::runtime_error(k + ": " + what), kind(k), diagnostics_json(diagnostics) {}
};

struct Artifact {
  std::string directory, artifact_path, manifest_json, diagnostics_json, code, requirements_json;
};

Artifact compile(const CudaSource& source, const CompileConfig& config);
void remove_artifact_directory(const std::string& directory);

}  // namespace trinity::host
