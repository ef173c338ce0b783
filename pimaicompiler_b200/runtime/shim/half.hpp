// Build shim: the reference's IR includes "half.hpp" (the half_float library, an un-vendored third-party header) only
// for a 16-bit storage type; libtorch's c10::Half serves.
#pragma once
#include <c10/util/Half.h>

namespace half_float {
using half = c10::Half;
}
