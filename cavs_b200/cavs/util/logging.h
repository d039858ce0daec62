// Minimal stand-in for the glog macros the reference's operators use
// (cavs/util/logging.h:8-10 defines the three verbosity levels).  CHECK and LOG(FATAL)
// print and abort, as glog does; VLOG output is enabled with the CAVS_V environment variable.
#ifndef CAVS_UTIL_LOGGING_H_
#define CAVS_UTIL_LOGGING_H_

#include <cstdlib>
#include <iostream>
#include <sstream>
#include <string>

#define V_TIMING 1
#define V_DEBUG 2
#define V_EXHAUSTIVE_DEBUG 3

namespace cavs_log {
enum Severity { INFO = 0, WARNING = 1, ERROR = 2, FATAL = 3 };
inline int Verbosity() {
  static int v = [] { const char* e = std::getenv("CAVS_V"); return e ? std::atoi(e) : 0; }();
  return v;
}
class Message {
 public:
  Message(const char* file, int line, Severity sev) : sev_(sev) { s_ << file << ":" << line << "] "; }
  ~Message() {
    std::cerr << s_.str() << std::endl;
    if (sev_ == FATAL) std::abort();
  }
  std::ostream& stream() { return s_; }
 private:
  std::ostringstream s_;
  Severity sev_;
};
struct Voidify { void operator&(std::ostream&) {} };
}  // namespace cavs_log

#define LOG(severity) ::cavs_log::Message(__FILE__, __LINE__, ::cavs_log::severity).stream()
#define CHECK(cond) \
  (cond) ? (void)0 : ::cavs_log::Voidify() & ::cavs_log::Message(__FILE__, __LINE__, ::cavs_log::FATAL).stream() << "Check failed: " #cond " "
#define CHECK_NOTNULL(p) (::cavs_log::CheckNotNull(__FILE__, __LINE__, #p, (p)))
#define VLOG_IS_ON(level) (::cavs_log::Verbosity() >= (level))
#define VLOG(level) \
  !VLOG_IS_ON(level) ? (void)0 : ::cavs_log::Voidify() & ::cavs_log::Message(__FILE__, __LINE__, ::cavs_log::INFO).stream()

namespace cavs_log {
template <typename T>
T CheckNotNull(const char* file, int line, const char* expr, T p) {
  if (p == nullptr) Message(file, line, FATAL).stream() << "Check failed: " << expr << " must not be NULL";
  return p;
}
}  // namespace cavs_log
#endif
