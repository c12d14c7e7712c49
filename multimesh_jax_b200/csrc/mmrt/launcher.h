// Native task launcher: a task body as a flat list of calls into the kernel library.
//
// The lowering turns a task template into `KernelCall` records: the address of an `extern "C"`
// entry point of the kernel library plus its packed arguments. Pointer arguments name a *slot*
// (a task input, a task output, the scratch tile, a persistent buffer) and a byte offset inside
// it, so one program serves every launch of the template: per launch the caller supplies only
// the slots' base addresses, the microbatch scalars and the stream, and `Launch` issues all
// kernels of the task without returning to the interpreter in between. This is the counterpart
// of the reference's task body binding tile pointers and scalar arguments to a compiled
// executable (src/pjrt_client/hlo_executor.cc:75-174) over a bump allocator on the cached
// scratch tile (src/pjrt_client/hlo_executor.cc:24-71).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace mmrt {

struct LaunchArg {
  enum Kind : int { kPtr = 0, kInt = 1, kFloat = 2, kStream = 3 };
  int kind = kInt;
  int slot = -1;              // kPtr: index into the base-address table
  int64_t value = 0;          // kPtr: byte offset; kInt: the value
  double fvalue = 0.0;        // kFloat
  int scalar = -1;            // kPtr: add scalars[scalar] * scalar_scale bytes (microbatch offsets)
  int64_t scalar_scale = 0;
};

struct KernelCall {
  uintptr_t fn = 0;
  std::string name;
  std::vector<LaunchArg> args;
};

class KernelProgram {
 public:
  static constexpr int kMaxIntArgs = 20;   // pointers, integers and the stream
  static constexpr int kMaxFloatArgs = 8;
  void AddCall(uintptr_t fn, const std::string& name, std::vector<LaunchArg> args);
  // Issues every call on `stream`. Returns 0, or a diagnostic in *error and a non-zero code
  // (the entry point's own return code when one of them refused its arguments).
  int Launch(const std::vector<uintptr_t>& bases, const std::vector<int64_t>& scalars, uintptr_t stream,
             std::string* error) const;
  size_t size() const { return calls_.size(); }
  std::string Describe() const;
  int64_t launches() const { return launches_; }

 private:
  std::vector<KernelCall> calls_;
  mutable int64_t launches_ = 0;
};

// A function with the calling convention of the kernel library, inside this module: used to
// test the launcher where no GPU exists. y[i] += a * x[i] for i < n; returns 0 (or 7 if n < 0).
extern "C" int mmrt_selftest_axpy(const float* x, float* y, int64_t n, float a, void* stream);

}  // namespace mmrt
