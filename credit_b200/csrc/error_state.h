// The per-thread error text behind credit_last_error(), for the translation units of
// the library that are not launch.cu.
#pragma once

namespace credit {

// Stores a printf-formatted message as the calling thread's last error and returns `code`.
int report_error(int code, const char* fmt, ...);

}  // namespace credit
