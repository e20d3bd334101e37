// standalone/core/types.h — the one type of the reference's vocabulary that the KV-cache interface
// needs, for builds OUTSIDE the reference tree only (this library itself, the stand-alone call-site
// program).  It sits in a directory of its own so that a build inside the reference tree, which puts
// only compat/ ahead of the reference's src/ on the include path, keeps resolving "core/types.h" and
// "compute/dispatch.h" to the reference's full headers.
// Numbering follows titan::DType (reference: src/core/types.h:17-33).
#pragma once

#include <cstddef>
#include <cstdint>

namespace titan {

enum class DType : uint8_t { FP32 = 0, FP16 = 1, BF16 = 2, FP8_E4M3 = 3 };

}  // namespace titan
