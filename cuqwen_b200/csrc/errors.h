// Error reporting shared by the translation units that export C-ABI entry points.
#pragma once

namespace cq {

// Stores a printf-style message as the calling thread's last error (cuqwen_last_error) and returns `code`.
int report_error(int code, const char* fmt, ...);

}  // namespace cq
