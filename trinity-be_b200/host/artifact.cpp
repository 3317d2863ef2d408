// Artifact builder: writes source.cu / exports.map, invokes the host compiler to produce
// program.so with exactly the five ABI symbols, and records manifest.json / diagnostics.json.
//
// Mirrors the reference's compile step (src/compile/cuda/mod.rs:24-118, :165-231) with one
// structural difference: kernels are compiled ahead of time into libtrinity_sm100.so, so the
// per-plan step compiles a host-only shim with the host C++ compiler instead of running nvcc
// over generated device code.
#include "artifact.hpp"

#include <sys/stat.h>
#include <sys/wait.h>
#include <unistd.h>

#include <array>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>

namespace trinity::host {

std::string g_library_dir;  // directory holding libtrinity_sm100.so (set through the C API)

namespace {

const char kExports[] =
    "{\n  global:\n    trinity_abi;\n    trinity_prepare;\n    trinity_launch;\n    trinity_status;\n"
    "    trinity_release;\n  local:\n    *;\n};\n";

void write_file(const std::string& path, const std::string& text) {
  std::ofstream out(path, std::ios::binary);
  if (!out || !(out << text)) throw CompileFailure("Io", "cannot write " + path, "");
}

struct RunResult {
  int exit_code;
  std::string output;
};
RunResult run(const std::vector<std::string>& argv) {
  // stdout and stderr are captured together through a pipe; no shell is involved.
  int fds[2];
  if (pipe(fds) != 0) throw CompileFailure("Io", "pipe failed", "");
  pid_t pid = fork();
  if (pid < 0) throw CompileFailure("Io", "fork failed", "");
  if (pid == 0) {
    dup2(fds[1], 1);
    dup2(fds[1], 2);
    close(fds[0]);
    close(fds[1]);
    std::vector<char*> args;
    for (auto& a : argv) args.push_back(const_cast<char*>(a.c_str()));
    args.push_back(nullptr);
    execvp(args[0], args.data());
    fprintf(stderr, "cannot execute %s: %s\n", args[0], strerror(errno));
    _exit(127);
  }
  close(fds[1]);
  RunResult r{0, ""};
  char buf[4096];
  ssize_t n;
  while ((n = read(fds[0], buf, sizeof buf)) > 0) r.output.append(buf, size_t(n));
  close(fds[0]);
  int status = 0;
  waitpid(pid, &status, 0);
  r.exit_code = WIFEXITED(status) ? WEXITSTATUS(status) : -1;
  return r;
}

std::string json_array(const std::vector<std::string>& items) {
  std::string s = "[";
  for (size_t i = 0; i < items.size(); ++i) s += (i ? "," : "") + ("\"" + json_escape(items[i]) + "\"");
  return s + "]";
}

std::string compiler_version(const std::string& compiler) {
  RunResult r = run({compiler, "--version"});
  if (r.exit_code != 0)
    throw CompileFailure("MissingCompiler", "host compiler " + compiler + " is not usable",
                         "{\"compiler\":\"" + json_escape(compiler) + "\",\"arguments\":[\"--version\"],\"exit_code\":" +
                             std::to_string(r.exit_code) + ",\"stdout\":\"\",\"stderr\":\"" + json_escape(r.output) + "\"}");
  return r.output.substr(0, r.output.find('\n'));
}

}  // namespace

Artifact compile(const CudaSource& source, const CompileConfig& config) {
  const std::string compiler = !config.host_compiler.empty() ? config.host_compiler
                               : getenv("CXX")               ? getenv("CXX")
                                                             : "g++";
  const std::string library_dir = !config.library_dir.empty() ? config.library_dir : g_library_dir;
  if (library_dir.empty()) throw CompileFailure("Config", "kernel library directory is not configured", "");
  struct stat st;
  if (stat((library_dir + "/libtrinity_sm100.so").c_str(), &st) != 0)
    throw CompileFailure("MissingLibrary", library_dir + "/libtrinity_sm100.so is missing; build it first", "");
  const std::string version = compiler_version(compiler);

  const char* tmp = getenv("TMPDIR");
  std::string pattern = std::string(tmp && *tmp ? tmp : "/tmp") + "/trinity-artifact-XXXXXX";
  std::vector<char> path(pattern.begin(), pattern.end());
  path.push_back('\0');
  if (!mkdtemp(path.data())) throw CompileFailure("Io", "cannot create an artifact directory", "");
  Artifact artifact;
  artifact.directory = path.data();
  artifact.artifact_path = artifact.directory + "/program.so";
  artifact.code = source.code;
  artifact.requirements_json = source.requirements_json;
  write_file(artifact.directory + "/source.cu", source.code);
  write_file(artifact.directory + "/exports.map", kExports);

  std::vector<std::string> argv = {
      compiler, "-shared", "-std=c++17", "-O2", "-fPIC", "-fvisibility=hidden", "-x", "c++",
      artifact.directory + "/source.cu", "-o", artifact.artifact_path,
      "-Wl,--version-script=" + artifact.directory + "/exports.map", "-Wl,-Bsymbolic-functions",
      "-L" + library_dir, "-ltrinity_sm100", "-Wl,-rpath," + library_dir};
  RunResult r = run(argv);
  std::ostringstream diagnostics;
  diagnostics << "{\"compiler\":\"" << json_escape(compiler) << "\",\"arguments\":"
              << json_array(std::vector<std::string>(argv.begin() + 1, argv.end())) << ",\"exit_code\":" << r.exit_code
              << ",\"stdout\":\"\",\"stderr\":\"" << json_escape(r.output) << "\"}";
  artifact.diagnostics_json = diagnostics.str();
  write_file(artifact.directory + "/diagnostics.json", artifact.diagnostics_json);
  if (r.exit_code != 0 || stat(artifact.artifact_path.c_str(), &st) != 0) {
    const std::string kind = r.exit_code != 0 ? "CompilerFailed" : "MissingArtifact";
    remove_artifact_directory(artifact.directory);
    throw CompileFailure(kind, "host compiler exited with " + std::to_string(r.exit_code), artifact.diagnostics_json);
  }
  std::ostringstream manifest;
  manifest << "{\"schema_version\":1,\"host_abi_version\":1,\"execution\":\"" << (source.persistent ? "persistent" : "streamed")
           << "\",\"library\":\"program.so\","
           << "\"source\":\"source.cu\",\"requirements\":" << source.requirements_json << ",\"toolchain\":{\"nvcc\":null,"
           << "\"cuda_major\":12,\"kernel_library\":\"" << json_escape(library_dir + "/libtrinity_sm100.so")
           << "\",\"cutlass\":null,\"nvshmem\":null,\"nvshmem_library_directory\":null,\"host_compiler\":\""
           << json_escape(version) << "\"}}";
  artifact.manifest_json = manifest.str();
  write_file(artifact.directory + "/manifest.json", artifact.manifest_json);
  return artifact;
}

void remove_artifact_directory(const std::string& directory) {
  if (directory.empty()) return;
  for (const char* name : {"source.cu", "exports.map", "program.so", "manifest.json", "diagnostics.json"})
    unlink((directory + "/" + name).c_str());
  rmdir(directory.c_str());
}

}  // namespace trinity::host
