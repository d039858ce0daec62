// Stand-in for the reference's glog wrapper (cavs/util/logging.h), used only to
// compile the reference's graph scheduler as a test oracle.  TEST INFRASTRUCTURE.
// CHECK aborts with a message; VLOG/LOG swallow their stream arguments.
#ifndef ORACLE_SHIM_CAVS_UTIL_LOGGING_H_
#define ORACLE_SHIM_CAVS_UTIL_LOGGING_H_
#include <cstdio>
#include <cstdlib>
#include <sstream>
#include <string>

#define V_TIMING 1
#define V_DEBUG 2
#define V_EXHAUSTIVE_DEBUG 3

namespace oracle_shim {
struct Sink {
  template <class T> Sink& operator<<(const T&) { return *this; }
};
struct Abort {
  std::ostringstream msg;
  Abort(const char* expr, const char* file, int line) { msg << file << ":" << line << " CHECK(" << expr << ") "; }
  ~Abort() { std::fprintf(stderr, "%s\n", msg.str().c_str()); std::abort(); }
  template <class T> Abort& operator<<(const T& v) { msg << v; return *this; }
};
}  // namespace oracle_shim

#define CHECK(cond) if (cond) {} else ::oracle_shim::Abort(#cond, __FILE__, __LINE__)
#define CHECK_NOTNULL(p) (p)
#define VLOG(level) if (true) {} else ::oracle_shim::Sink()
#define VLOG_IS_ON(level) false
#define LOG(severity) ::oracle_shim::Sink()
#endif
