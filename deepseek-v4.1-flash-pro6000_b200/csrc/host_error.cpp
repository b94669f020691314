#include "host_error.h"
#include <string>
namespace ds41 {
namespace {
thread_local std::string message_store;
}
void set_error(const char *message) { message_store = message ? message : ""; }
const char *last_error() { return message_store.c_str(); }
}  // namespace ds41
