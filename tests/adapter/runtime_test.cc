// The device test of the reference (pjrt_plugin/src/runtime_test.cc:136-267: blob A two-level
// elementwise, blob B on-device WHILE, blob C GELU map-region) driven through the adapter classes:
// OclRuntime::Create -> VmProgram::Parse -> LoadedProgram::Load -> Execute (host in / host out),
// then ExecuteDevice on the same program. The blobs, inputs and expected outputs are files
// written by the calling test (tests/kat_programs.py builds them):
//   <dir>/<case>.blob, <dir>/<case>.in<i>, <dir>/<case>.want<o>    (f32 data)
// usage: runtime_test <dir> <case>:<n_in>:<n_out>:<rtol> ...
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>

#include "b2_runtime_adapter.h"

static std::vector<uint8_t> slurp(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) { std::cerr << "cannot open " << path << "\n"; std::exit(2); }
  return std::vector<uint8_t>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}

static bool close_f32(const std::vector<uint8_t>& got, const std::vector<uint8_t>& want, double rtol, const std::string& what) {
  if (got.size() != want.size()) { std::cerr << what << ": size " << got.size() << " != " << want.size() << "\n"; return false; }
  const float* g = reinterpret_cast<const float*>(got.data());
  const float* w = reinterpret_cast<const float*>(want.data());
  for (size_t i = 0; i < got.size() / 4; ++i) {
    if (!(std::fabs(double(g[i]) - double(w[i])) <= rtol * std::fabs(double(w[i])) + rtol)) {
      std::cerr << what << ": element " << i << " got " << g[i] << " want " << w[i] << "\n";
      return false;
    }
  }
  return true;
}

int main(int argc, char** argv) {
  if (argc < 3) { std::cerr << "usage: runtime_test <dir> <case>:<n_in>:<n_out>:<rtol> ...\n"; return 2; }
  const std::string dir = argv[1];
  std::string err;
  auto rt = pjrt_ocl::OclRuntime::Create(&err);
  if (!rt) { std::cerr << "OclRuntime::Create: " << err << "\n"; return 1; }
  std::cout << "device " << rt->info().name << ", " << rt->ngroups() << " lanes, ew_ts " << rt->ew_ts() << ", mma_t " << rt->mma_t() << "\n";
  int failed = 0;
  for (int a = 2; a < argc; ++a) {
    std::string name; int n_in = 0, n_out = 0; double rtol = 0;
    {
      std::stringstream ss(argv[a]); std::string tok;
      std::getline(ss, name, ':'); std::getline(ss, tok, ':'); n_in = std::stoi(tok);
      std::getline(ss, tok, ':'); n_out = std::stoi(tok); std::getline(ss, tok, ':'); rtol = std::stod(tok);
    }
    const auto blob = slurp(dir + "/" + name + ".blob");
    pjrt_ocl::VmProgram prog;
    if (!pjrt_ocl::VmProgram::Parse(blob.data(), blob.size(), &prog, &err)) { std::cerr << name << ": Parse: " << err << "\n"; ++failed; continue; }
    if (int(prog.num_inputs()) != n_in || int(prog.num_outputs()) != n_out) { std::cerr << name << ": arity\n"; ++failed; continue; }
    auto lp = pjrt_ocl::LoadedProgram::Load(rt.get(), std::move(prog), &err);
    if (!lp) { std::cerr << name << ": Load: " << err << "\n"; ++failed; continue; }
    std::vector<std::vector<uint8_t>> ins(n_in), want(n_out), got;
    std::vector<const void*> in_ptrs(n_in);
    for (int i = 0; i < n_in; ++i) { ins[i] = slurp(dir + "/" + name + ".in" + std::to_string(i)); in_ptrs[i] = ins[i].data(); }
    for (int o = 0; o < n_out; ++o) want[o] = slurp(dir + "/" + name + ".want" + std::to_string(o));
    bool ok = lp->Execute(in_ptrs, &got, &err);
    if (!ok) { std::cerr << name << ": Execute: " << err << "\n"; ++failed; continue; }
    for (int o = 0; o < n_out; ++o) ok = close_f32(got[o], want[o], rtol, name + " Execute out " + std::to_string(o)) && ok;
    // the plugin's path: device buffers in, pooled device buffers out. A fresh load: blob B counts in a
    // constant buffer, which (here as in the reference, runtime.cc:1066) is uploaded at Load only.
    pjrt_ocl::VmProgram prog2;
    if (!pjrt_ocl::VmProgram::Parse(blob.data(), blob.size(), &prog2, &err)) { std::cerr << name << ": Parse: " << err << "\n"; ++failed; continue; }
    lp = pjrt_ocl::LoadedProgram::Load(rt.get(), std::move(prog2), &err);
    if (!lp) { std::cerr << name << ": Load: " << err << "\n"; ++failed; continue; }
    std::vector<void*> din(n_in), dout;
    for (int i = 0; i < n_in; ++i) {
      din[i] = rt->AllocDevice(ins[i].size() < 16 ? 16 : ins[i].size(), &err);
      if (!din[i] || !rt->WriteToDevice(din[i], ins[i].data(), ins[i].size(), &err)) { std::cerr << name << ": upload: " << err << "\n"; ok = false; }
    }
    if (ok && !lp->ExecuteDevice(din, &dout, &err)) { std::cerr << name << ": ExecuteDevice: " << err << "\n"; ok = false; }
    for (int o = 0; ok && o < n_out; ++o) {
      std::vector<uint8_t> back(want[o].size());
      ok = rt->ReadFromDevice(back.data(), dout[o], back.size(), &err) && close_f32(back, want[o], rtol, name + " ExecuteDevice out " + std::to_string(o));
      rt->PoolFree(dout[o], back.size());
    }
    for (int i = 0; i < n_in; ++i) if (din[i]) rt->PoolFree(din[i], ins[i].size() < 16 ? 16 : ins[i].size());
    std::cout << (ok ? "PASS " : "FAIL ") << name << "\n";
    if (!ok) ++failed;
  }
  return failed ? 1 : 0;
}
