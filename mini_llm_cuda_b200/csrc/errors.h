// Thread-local error message shared by the translation units of the library.
#pragma once
namespace mlb {
// Stores the formatted message for mlb_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);
}  // namespace mlb
