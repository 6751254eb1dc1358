/* Stand-in for <glog/logging.h>, which the reference includes from src/logging.h but which is
 * not installed here.  Test infrastructure only (used to compile the reference's own CUDA
 * sources into oracle/_ref/).  Failed checks throw instead of aborting the process, so that a
 * test can report them. */
#pragma once
#include <sstream>
#include <stdexcept>
#include <string>

namespace gs_ref_shim {
struct Thrower {
  std::ostringstream os;
  bool fatal;
  explicit Thrower(bool f) : fatal(f) {}
  template <typename T>
  Thrower& operator<<(const T& v) { os << v; return *this; }
  ~Thrower() noexcept(false) { if (fatal) throw std::runtime_error(os.str()); }
};
struct Voidify { void operator&(Thrower&) {} };
}  // namespace gs_ref_shim

#define GS_SHIM_FATAL gs_ref_shim::Thrower(true)
#define GS_SHIM_INFO gs_ref_shim::Thrower(false)
#define LOG(severity) GS_SHIM_LOG_##severity
#define GS_SHIM_LOG_FATAL GS_SHIM_FATAL << "[FATAL] "
#define GS_SHIM_LOG_ERROR GS_SHIM_INFO
#define GS_SHIM_LOG_WARNING GS_SHIM_INFO
#define GS_SHIM_LOG_INFO GS_SHIM_INFO
#define CHECK(cond) (cond) ? (void)0 : gs_ref_shim::Voidify() & GS_SHIM_FATAL << "Check failed: " #cond " "
#define GS_SHIM_CHECK_OP(a, b, op) CHECK((a)op(b))
#define CHECK_EQ(a, b) GS_SHIM_CHECK_OP(a, b, ==)
#define CHECK_NE(a, b) GS_SHIM_CHECK_OP(a, b, !=)
#define CHECK_LE(a, b) GS_SHIM_CHECK_OP(a, b, <=)
#define CHECK_LT(a, b) GS_SHIM_CHECK_OP(a, b, <)
#define CHECK_GE(a, b) GS_SHIM_CHECK_OP(a, b, >=)
#define CHECK_GT(a, b) GS_SHIM_CHECK_OP(a, b, >)
#define CHECK_NOTNULL(p) (p)
#define DCHECK(cond) CHECK(cond)
#define DCHECK_EQ(a, b) CHECK_EQ(a, b)
#define DCHECK_NE(a, b) CHECK_NE(a, b)
#define DCHECK_LE(a, b) CHECK_LE(a, b)
#define DCHECK_LT(a, b) CHECK_LT(a, b)
#define DCHECK_GE(a, b) CHECK_GE(a, b)
#define DCHECK_GT(a, b) CHECK_GT(a, b)
#define VLOG(n) GS_SHIM_INFO
