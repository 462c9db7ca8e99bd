/* Stand-in for dragon/core/types.h when the reference's converters and CPU
 * optimizer loops are compiled on their own (TEST INFRASTRUCTURE ONLY).
 *
 * The real header drags in generated protobuf code; the files compiled here
 * (dragon/utils/conversions.h, dragon/kernels/training/cpu/{adam,sgd}_kernel.cc)
 * only need the two 16-bit storage types, which the reference declares as
 * structs holding one `unsigned short x` (dragon/core/types.h:36-42). */
#ifndef ORACLE_REF_STUB_TYPES_H_
#define ORACLE_REF_STUB_TYPES_H_

#include <cmath>
#include <cstdint>
#include <cstring>

namespace dragon {
struct alignas(2) float16 { unsigned short x; };
struct alignas(2) bfloat16 { unsigned short x; };
}  // namespace dragon

#endif
