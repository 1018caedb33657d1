// intrinsics.h -- the CPU platforms define their microkernel macros here
// (FLOAT_CONV_TILE_C and friends, docs/Defining_Platforms.md).  On the B200 platform the
// microkernels are CUDA kernels inside libsmall_b200.so, reached through the C ABI
// (include/small_b200.h), so there is nothing to define for the host compiler.
#pragma once
#include <small_b200.h>
