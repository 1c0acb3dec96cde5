// Error reporting shared by the host-side translation units. The reference reports
// failures by throwing std::runtime_error from fail() (src/model/impl/common.h:48); at a
// C boundary the same message is kept per thread and a negative status is returned.
#pragma once

#include <cstdarg>
#include <cstdio>

#include "../../include/espetero_attn.h"

namespace esp {

inline char* last_error_buffer() {
  static thread_local char buf[512] = "";
  return buf;
}

#if defined(__GNUC__)
__attribute__((format(printf, 2, 3)))
#endif
inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  std::vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

}  // namespace esp
