// Stand-in for <glog/logging.h>, which is not installed here: LOG(x) and VLOG(n) swallow what is streamed
// into them.  lumia431/photon_infer uses glog for progress and debug lines only (no CHECK, no flags), so
// its code compiles unchanged against this header and computes the same.
#pragma once
#include <ostream>

namespace photon_glog_shim {
struct NullStream {
  template <typename T> NullStream& operator<<(const T&) { return *this; }
  NullStream& operator<<(std::ostream& (*)(std::ostream&)) { return *this; }
};
}  // namespace photon_glog_shim

#define LOG(severity) ::photon_glog_shim::NullStream()
#define VLOG(level) ::photon_glog_shim::NullStream()
#define VLOG_IS_ON(level) false

static int FLAGS_logtostderr = 0;      // the demos set it; nothing reads it here

namespace google {
inline void InitGoogleLogging(const char*) {}
inline void ShutdownGoogleLogging() {}
}  // namespace google
