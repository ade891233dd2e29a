#include "errors.h"

#include "../api.h"

namespace tileccl {
namespace {
thread_local std::string g_last_error;
}
void set_last_error(const std::string& msg) { g_last_error = msg; }
const std::string& last_error() { return g_last_error; }
}  // namespace tileccl

extern "C" const char* tccl_last_error(void) { return tileccl::last_error().c_str(); }
extern "C" const char* tccl_version(void) { return "0.1.0-b200"; }
