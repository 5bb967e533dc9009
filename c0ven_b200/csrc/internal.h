// What the library's translation units share beside the public header.
#pragma once

#include <string>

namespace moe {

// The text moe_last_error(NULL) returns on this thread: for calls that fail before there is a layer to keep it in.
void set_create_error(const std::string &message);

}  // namespace moe
