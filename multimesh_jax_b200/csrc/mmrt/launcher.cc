#include "launcher.h"

#include <sstream>
#include <stdexcept>

namespace mmrt {

#if !defined(__x86_64__) && !defined(__aarch64__)
#error "the uniform trampoline below relies on the x86-64 System V / AArch64 procedure call standards"
#endif

namespace {
// Every entry point of the kernel library takes pointers, 32- or 64-bit integers, floats and a
// stream and returns int. Under both supported calling conventions the k-th integer-class
// argument travels in the k-th integer register (then on the stack, in order) and the k-th
// float in the k-th vector register, independently of how the two kinds interleave, and a
// callee reads only the low half of a register that carries a 32-bit integer. One signature
// with all integer-class arguments first therefore calls any of them; surplus arguments are
// ignored by the callee.
using Uniform = int (*)(int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                        int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                        float, float, float, float, float, float, float, float);
}  // namespace

void KernelProgram::AddCall(uintptr_t fn, const std::string& name, std::vector<LaunchArg> args) {
  if (!fn) throw std::runtime_error("native launcher: entry point '" + name + "' has no address");
  int ni = 0, nf = 0;
  for (auto& a : args) (a.kind == LaunchArg::kFloat ? nf : ni)++;
  if (ni > kMaxIntArgs || nf > kMaxFloatArgs)
    throw std::runtime_error("native launcher: too many arguments for '" + name + "'");
  KernelCall c;
  c.fn = fn;
  c.name = name;
  c.args = std::move(args);
  calls_.push_back(std::move(c));
}

int KernelProgram::Launch(const std::vector<uintptr_t>& bases, const std::vector<int64_t>& scalars, uintptr_t stream,
                          std::string* error) const {
  for (size_t k = 0; k < calls_.size(); ++k) {
    const KernelCall& c = calls_[k];
    int64_t iv[kMaxIntArgs] = {};
    float fv[kMaxFloatArgs] = {};
    int ni = 0, nf = 0;
    for (const LaunchArg& a : c.args) {
      switch (a.kind) {
        case LaunchArg::kPtr: {
          if (a.slot < 0) { iv[ni++] = 0; break; }      // a null pointer argument
          if (a.slot >= static_cast<int>(bases.size()) || bases[a.slot] == 0) {
            if (error) *error = "call " + std::to_string(k) + " (" + c.name + "): slot " + std::to_string(a.slot) + " has no address";
            return -1;
          }
          int64_t addr = static_cast<int64_t>(bases[a.slot]) + a.value;
          if (a.scalar >= 0) {
            if (a.scalar >= static_cast<int>(scalars.size())) {
              if (error) *error = "call " + std::to_string(k) + " (" + c.name + "): missing scalar " + std::to_string(a.scalar);
              return -1;
            }
            addr += scalars[a.scalar] * a.scalar_scale;
          }
          iv[ni++] = addr;
          break;
        }
        case LaunchArg::kInt: iv[ni++] = a.value; break;
        case LaunchArg::kStream: iv[ni++] = static_cast<int64_t>(stream); break;
        case LaunchArg::kFloat: fv[nf++] = static_cast<float>(a.fvalue); break;
      }
    }
    const int rc = reinterpret_cast<Uniform>(c.fn)(iv[0], iv[1], iv[2], iv[3], iv[4], iv[5], iv[6], iv[7], iv[8], iv[9],
                                                   iv[10], iv[11], iv[12], iv[13], iv[14], iv[15], iv[16], iv[17], iv[18],
                                                   iv[19], fv[0], fv[1], fv[2], fv[3], fv[4], fv[5], fv[6], fv[7]);
    ++launches_;
    if (rc != 0) {
      if (error) *error = "call " + std::to_string(k) + " (" + c.name + ") returned " + std::to_string(rc);
      return rc;
    }
  }
  return 0;
}

std::string KernelProgram::Describe() const {
  std::ostringstream os;
  for (size_t k = 0; k < calls_.size(); ++k) {
    os << k << ": " << calls_[k].name << "(";
    for (size_t i = 0; i < calls_[k].args.size(); ++i) {
      const LaunchArg& a = calls_[k].args[i];
      if (i) os << ", ";
      if (a.kind == LaunchArg::kPtr) {
        if (a.slot < 0) os << "null";
        else {
          os << "s" << a.slot << "+" << a.value;
          if (a.scalar >= 0) os << "+x" << a.scalar << "*" << a.scalar_scale;
        }
      } else if (a.kind == LaunchArg::kInt) os << a.value;
      else if (a.kind == LaunchArg::kFloat) os << a.fvalue << "f";
      else os << "stream";
    }
    os << ")\n";
  }
  return os.str();
}

extern "C" int mmrt_selftest_axpy(const float* x, float* y, int64_t n, float a, void*) {
  if (n < 0) return 7;
  for (int64_t i = 0; i < n; ++i) y[i] += a * x[i];
  return 0;
}

}  // namespace mmrt
