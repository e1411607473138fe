// Shared definitions of the reference-named C++ API (the part of DUQLinear4bitCUDA's
// include/common.h and include/int4.h that callers of gemm.h / quant.h rely on):
// the int4 storage type and the clamp bounds. No CUTLASS dependency.
#pragma once
#include <cstdint>

// Two 4-bit values per byte, element 2j in the low nibble (include/int4.h:254-266 of the reference).
using Int4Storage = uint8_t;
using UInt4Storage = uint8_t;
constexpr unsigned kElementsPerVector = 2;
constexpr unsigned kElementsPerVectorUInt4 = 2;

// Clamp bounds (include/common.h:53-57 of the reference). There qmax_sym is written
// `(7 - 1e-8)`, an int initialised from a double just below 7: it is 6, and symmetric codes
// never exceed 6. The kernels of this library use the same bound.
constexpr int qmin_sym = -8;
constexpr int qmax_sym = 6;
constexpr int qmin_asym = 0;
constexpr int qmax_asym = 15;
