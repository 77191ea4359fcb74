// Error classes and small utilities of the host runtime.
//
// The reference distinguishes two failure classes (include/utils/logging.h:96-148,301-340):
// VERIFY* raises std::logic_error (the model or the input is at fault; C-ABI status 1) and
// CHECK* / LOG(FATAL) raises std::runtime_error (status 2).  The same split is kept here so that
// every malformed model maps to the status the reference returns.
#pragma once
#include <cstdint>
#include <cstdlib>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace cvm {

// Environment variables that re-route operators exist for experiments only: honoured in builds
// made with -DCVM_B200_DEV_SWITCHES, ignored by the shipped library.
inline const char* dev_env(const char* name) {
#ifdef CVM_B200_DEV_SWITCHES
  return getenv(name);
#else
  (void)name;
  return nullptr;
#endif
}

struct ParamError : public std::runtime_error {
  explicit ParamError(const std::string& s) : std::runtime_error(s) {}
};

template <typename E>
class Thrower {
 public:
  Thrower(const char* file, int line, const char* cond) {
    const char* base = file;
    for (const char* p = file; *p; ++p)
      if (*p == '/') base = p + 1;
    os_ << base << ":" << line << ": ";
    if (cond) os_ << "Check failed: " << cond << " ";
  }
  std::ostringstream& stream() { return os_; }
  ~Thrower() noexcept(false) { throw E(os_.str()); }

 private:
  std::ostringstream os_;
};

#define VERIFY(c) \
  if (c) {} else ::cvm::Thrower<std::logic_error>(__FILE__, __LINE__, #c).stream()
#define VERIFY_EQ(a, b) VERIFY((a) == (b))
#define VERIFY_NE(a, b) VERIFY((a) != (b))
#define VERIFY_LT(a, b) VERIFY((a) < (b))
#define VERIFY_LE(a, b) VERIFY((a) <= (b))
#define VERIFY_GT(a, b) VERIFY((a) > (b))
#define VERIFY_GE(a, b) VERIFY((a) >= (b))
#define CHECK(c) \
  if (c) {} else ::cvm::Thrower<std::runtime_error>(__FILE__, __LINE__, #c).stream()
#define CHECK_EQ(a, b) CHECK((a) == (b))
#define FATAL() ::cvm::Thrower<std::runtime_error>(__FILE__, __LINE__, nullptr).stream()

typedef std::vector<int64_t> Shape;

// A refusal this library adds on top of the reference's checks (a model the reference would run
// with out-of-bounds reads).  It is raised only after every check of the reference has passed, so
// a model the reference refuses keeps the reference's status class.
inline std::string& deferred_refusal() {
  static thread_local std::string text;
  return text;
}

inline int64_t shape_size(const Shape& s) {
  int64_t n = 1;
  for (auto d : s) n *= d;
  return n;
}
inline std::string shape_str(const Shape& s) {
  std::ostringstream os;
  os << "[";
  for (size_t i = 0; i < s.size(); ++i) os << (i ? "," : "") << s[i];
  os << "]";
  return os.str();
}

// Bits needed to hold a sum of `size` terms (src/top/op_common.h:277-281).
inline int reduce_sum_bits(int64_t size) {
  int prec = 0;
  while (size != 0) { prec++; size >>= 1; }
  return prec;
}
// Precision of the number n: smallest p with |n| <= 2^(p-1)-1 (src/top/op_common.h:294-299).
inline int number_precision(int64_t n) {
  int prec = 0;
  n = n + 1;
  while (n != 0) { prec++; n >>= 1; }
  return prec + 1;
}

}  // namespace cvm
