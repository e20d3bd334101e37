// core/types.h — the one type of the reference's vocabulary that the KV-cache interface
// needs, for builds outside the reference tree.  Inside the reference tree its own
// src/core/types.h is found first on the include path and this file is not used.
// Numbering follows titan::DType (reference: src/core/types.h:17-33).
#pragma once

#include <cstddef>
#include <cstdint>

namespace titan {

enum class DType : uint8_t { FP32 = 0, FP16 = 1, BF16 = 2, FP8_E4M3 = 3 };

}  // namespace titan
