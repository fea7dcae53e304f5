// The builds of the megakernel the library carries. Each is the same interpreter
// (vm_kernel.cu) compiled with only some tile-op families present; a program runs
// on the first build in this list that has every family its tasks use, so it does
// not pay (in registers, instruction-cache footprint and compiler decisions) for
// tile ops it never executes. The reference builds its megakernel with a
// compile-time op mask for attribution (VMO_STUB_MASK,
// pjrt_plugin/kernels/vm_main.cl:19-27); here the mask selects what is shipped.
//
// B2_VARIANT_LIST(X) expands X(name, family mask) in order of preference
// (smallest first; the last one holds everything). The build script reads the
// same list to compile one object per entry.
#ifndef B2VM_VARIANTS_H_
#define B2VM_VARIANTS_H_

#include "format.h"

#define B2_FAMS_STREAM (b2::kFamEw | b2::kFamMove | b2::kFamRed | b2::kFamRows | b2::kFamRegion)
#define B2_VARIANT_LIST(X)                               \
  X(stream, B2_FAMS_STREAM)                              \
  X(shortrun, B2_FAMS_STREAM | b2::kFamShort)            \
  X(matmul, B2_FAMS_STREAM | b2::kFamMma)                \
  X(attn, B2_FAMS_STREAM | b2::kFamMma | b2::kFamFlash)  \
  X(all, b2::kFamAll)

#endif
