// Forwarding header: CuQwen sources say #include "load_weights.h"; with -I<this directory> they get the source-compatible
// declarations of cuqwen_compat.hpp (same types, macros and functions on top of the C ABI of cuqwen_b200.h).
#pragma once
#include "../cuqwen_compat.hpp"
